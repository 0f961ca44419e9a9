"""The CPU oracle's transformer forwards against logits computed by an independent implementation.

tests/golden/hf_forward_golden.npz (made by tests/golden/make_hf_golden.py) holds small seeded Llama, Qwen2 and GPT-2
networks under their GGUF tensor names together with the logits Hugging Face `transformers` computes for them in
float64.  wgml's own tests hold no numeric vectors for the forward pass (only GPU-vs-CPU self-checks), so this is what
anchors the oracle's reading of the architectures: RoPE pairing (Original for Llama files, Neox for Qwen2) and
frequencies, grouped-query head mapping, attention scaling, SwiGLU, q/k/v biases, GPT-2's fused qkv, learned
positions, tanh GELU and the tied output head.  Tolerance: the oracle sums in f32, the fixture in f64."""
import os

import numpy as np
import pytest

import oracle
from wgml_b200 import synth

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hf_forward_golden.npz")
RTOL, ATOL = 2e-5, 2e-5   # f32 sums against f64 sums; logits of order 1-10


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def _net(golden, name):
    cfg = {k.split("/")[-1]: golden[k].item() for k in golden.files if k.startswith(f"{name}/cfg/")}
    cfg = {k: (float(v) if k in ("rope_base_freq", "rms_norm_eps") else int(v)) for k, v in cfg.items()}
    tensors = {k[len(name) + 3:]: (synth.F32, golden[k].astype(np.float32)) for k in golden.files if k.startswith(f"{name}/w/")}
    return cfg, tensors, golden[f"{name}/tokens"], golden[f"{name}/logits"]


@pytest.mark.parametrize("name,rope_variant", [("llama", 0), ("qwen2", 1)])
def test_llama_family_logits_match_transformers(golden, name, rope_variant):
    cfg, tensors, tokens, want = _net(golden, name)
    m = oracle.Llama2Oracle(cfg, tensors, rope_variant=rope_variant)
    for pos, tok in enumerate(tokens):
        got = m.forward(int(tok), pos)
        np.testing.assert_allclose(got, want[pos], rtol=RTOL, atol=ATOL, err_msg=f"{name}, position {pos}")
    assert int(np.argmax(got)) == int(np.argmax(want[-1]))


def test_rope_variant_matters(golden):
    """The check above has teeth: the same Llama weights under the other RoPE pairing give other logits."""
    cfg, tensors, tokens, want = _net(golden, "llama")
    m = oracle.Llama2Oracle(cfg, tensors, rope_variant=1)
    for pos, tok in enumerate(tokens):
        got = m.forward(int(tok), pos)
    assert np.abs(got - want[-1]).max() > 100 * ATOL


def test_gpt2_logits_match_transformers(golden):
    cfg, tensors, tokens, want = _net(golden, "gpt2")
    m = oracle.Gpt2Oracle(cfg, tensors)
    for pos, tok in enumerate(tokens):
        got = m.forward(int(tok), pos)
        np.testing.assert_allclose(got, want[pos], rtol=RTOL, atol=ATOL, err_msg=f"gpt2, position {pos}")
