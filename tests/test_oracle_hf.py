"""The CPU oracle's transformer forwards against logits computed by an independent implementation.

tests/golden/hf_forward_golden.npz (made by tests/golden/make_hf_golden.py) holds the logits Hugging Face
`transformers` computes in float64 for seeded Llama, Qwen2 and GPT-2 networks.  wgml's own tests hold no numeric
vectors for the forward pass (only GPU-vs-CPU self-checks), so this is what anchors the oracle's reading of the
architectures: RoPE pairing (Original for Llama files, Neox for Qwen2) and frequencies, grouped-query head mapping,
attention scaling, SwiGLU, q/k/v biases, GPT-2's fused qkv, learned positions, tanh GELU and the tied output head.
Tolerance: the oracle sums in f32, the fixture in f64."""
import numpy as np
import pytest

import oracle
from hf_golden import network

TOL = 2e-5   # relative, and absolute in units of the largest logit


def _check(got, want, what):
    np.testing.assert_allclose(got, want, rtol=TOL, atol=TOL * max(1.0, float(np.abs(want).max())), err_msg=what)


@pytest.mark.parametrize("name,rope_variant", [("llama", 0), ("qwen2", 1)])
def test_llama_family_logits_match_transformers(name, rope_variant):
    cfg, tensors, tokens, want = network(name)
    m = oracle.Llama2Oracle(cfg, tensors, rope_variant=rope_variant)
    for pos, tok in enumerate(tokens):
        got = m.forward(int(tok), pos)
        _check(got, want[pos], f"{name}, position {pos}")
    assert int(np.argmax(got)) == int(np.argmax(want[-1]))


def test_rope_variant_matters():
    """The check above has teeth: the same Llama weights under the other RoPE pairing give other logits."""
    cfg, tensors, tokens, want = network("llama")
    m = oracle.Llama2Oracle(cfg, tensors, rope_variant=1)
    for pos, tok in enumerate(tokens):
        got = m.forward(int(tok), pos)
    assert np.abs(got - want[-1]).max() > 1000 * TOL


def test_gpt2_logits_match_transformers():
    cfg, tensors, tokens, want = network("gpt2")
    m = oracle.Gpt2Oracle(cfg, tensors)
    for pos, tok in enumerate(tokens):
        _check(m.forward(int(tok), pos), want[pos], f"gpt2, position {pos}")
