"""Access to tests/golden/hf_forward_golden.npz for the CPU and GPU tests: the seeded networks (drawn again with the
generator's own numpy code, checked against the stored checksum) and the logits Hugging Face `transformers` computed."""
import importlib.util
import os

import numpy as np

from wgml_b200 import synth

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _generator():
    spec = importlib.util.spec_from_file_location("make_hf_golden", os.path.join(GOLDEN_DIR, "make_hf_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)   # numpy only; transformers is imported inside the functions that run it
    return mod


def network(name: str):
    """(config, {tensor name: (F32, array)}, token ids, expected logits [position][vocab]) of 'llama', 'qwen2' or 'gpt2'."""
    gen = _generator()
    golden = np.load(os.path.join(GOLDEN_DIR, "hf_forward_golden.npz"))
    cfg, t, tokens = gen.draw_gpt2() if name == "gpt2" else gen.draw_llama(name)
    assert gen.checksum(t) == int(golden[f"{name}/weights_crc32"]), \
        "numpy draws other weights than when the fixture was made: run tests/golden/make_hf_golden.py again"
    assert np.array_equal(tokens, golden[f"{name}/tokens"])
    return cfg, {k: (synth.F32, v) for k, v in t.items()}, tokens, golden[f"{name}/logits"]
