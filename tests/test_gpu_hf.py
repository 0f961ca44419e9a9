"""The CUDA Llama-2 / Qwen2 / GPT-2 models against logits computed by an independent implementation.

Same fixture as tests/test_oracle_hf.py (Hugging Face `transformers`, float64, seeded networks; made by
tests/golden/make_hf_golden.py), here through the C ABI on the device: 1e-3 relative / 1e-4 absolute, the absolute
term in units of the largest logit, for the fused and the dispatch-by-dispatch schedules."""
import numpy as np
import pytest

from conftest import ATOL, RTOL, assert_close
from hf_golden import network
from wgml_b200.models import Gpt2, Gpt2Params, Llama2, Llama2Config, LlamaModelType

pytestmark = pytest.mark.gpu


def _walk(model, tokens, want, what):
    for pos, tok in enumerate(tokens):
        model.dispatch(int(tok), pos)
        got = model.logits().cpu().numpy()
        assert_close(got, want[pos], RTOL, ATOL * max(1.0, float(np.abs(want[pos]).max())), f"{what} logits at position {pos}")
    assert int(np.argmax(got)) == int(np.argmax(want[-1]))


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("name", ["llama", "qwen2"])
def test_llama_family_logits_match_transformers(name, fused):
    cfg, tensors, tokens, want = network(name)
    c = Llama2Config(cfg["dim"], cfg["hidden_dim"], cfg["n_layers"], cfg["n_q_heads"], cfg["n_kv_heads"], cfg["vocab_size"],
                     cfg["seq_len"], cfg["rope_base_freq"], cfg["rms_norm_eps"])
    m = Llama2(c, LlamaModelType.Qwen2 if name == "qwen2" else LlamaModelType.Llama)
    m.load_tensors(tensors)
    m.set_fused(fused)
    _walk(m, tokens, want, f"{name} (fused={fused})")
    m.close()


@pytest.mark.parametrize("fused", [True, False])
def test_gpt2_logits_match_transformers(fused):
    cfg, tensors, tokens, want = network("gpt2")
    m = Gpt2(Gpt2Params(cfg["n_vocab"], cfg["n_seq"], cfg["n_embd"], cfg["n_head"], cfg["n_layer"], cfg["ff_len"], 3 * cfg["n_embd"], 7))
    m.load_tensors(tensors)
    m.set_fused(fused)
    _walk(m, tokens, want, f"gpt2 (fused={fused})")
    m.close()
