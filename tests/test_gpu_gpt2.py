"""GPT-2 forward and token loop against the CPU transformer (oracle)."""
import numpy as np
import pytest

from conftest import ATOL, RTOL, assert_close
from helpers import SMALL_GPT2, gpt2_pair
from wgml_b200 import synth

pytestmark = pytest.mark.gpu


def compare_steps(gpu, cpu, tokens, what=""):
    for i, tok in enumerate(tokens):
        gpu.dispatch(int(tok), i)
        exp = cpu.forward(int(tok), i)
        scale = max(1.0, float(np.abs(exp).max()))
        assert_close(gpu.logits().cpu().numpy(), exp, RTOL, ATOL * scale, f"{what} logits at step {i}")
    kc, vc = cpu.caches()
    n = len(tokens)
    for l in range(gpu.params.n_layer):
        assert_close(gpu.key_cache(l)[:n].cpu().numpy(), kc[l, :n], RTOL, ATOL * max(1.0, float(np.abs(kc[l, :n]).max())), "key cache")
        assert_close(gpu.value_cache(l)[:n].cpu().numpy(), vc[l, :n], RTOL, ATOL * max(1.0, float(np.abs(vc[l, :n]).max())), "value cache")


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("qtype", [synth.Q8_0, synth.F32, synth.Q5_1])
def test_small_gpt2(fused, qtype):
    cfg = dict(SMALL_GPT2, default_qtype=qtype)
    gpu, cpu, _ = gpt2_pair(cfg, seed=1, fused=fused, scale=0.002)
    prompt = synth.prompt(10, cfg["n_vocab"], 1)
    compare_steps(gpu, cpu, prompt, what=f"gpt2 {qtype}")
    gpu2, cpu2, _ = gpt2_pair(cfg, seed=1, fused=fused, scale=0.002)
    exp = cpu2.decode(prompt, 32)
    assert np.array_equal(gpu2.decode(prompt, 32), exp)


def test_gpt2_124m_shapes_two_layers():
    """GPT-2 124M dimensions (768, 12 heads, FFN 3072, ctx 1024, vocab 50257 -- an odd row count) in
    Q8_0 with 2 layers."""
    cfg = dict(synth.CONFIGS["gpt2-124m"], n_layer=2)
    gpu, cpu, _ = gpt2_pair(cfg, seed=2, scale=0.001)
    prompt = synth.prompt(6, cfg["n_vocab"], 2)
    compare_steps(gpu, cpu, prompt, what="gpt2-124m-2l")
    exp = cpu.decode(prompt[:3], 8, 0)  # overwrites positions 0.. of both caches identically
    assert np.array_equal(gpu.decode(prompt[:3], 8), exp)


@pytest.mark.parametrize("fused", [True, False])
def test_gpt2_124m_full_depth(fused):
    """The whole GPT-2 124M configuration (12 layers, Q8_0), weights scaled so that pre-activations stay of
    order one (at the scale of the timing configuration a random 12-layer network amplifies f32 rounding
    differences ~3x per layer and implementations cannot be compared): logits along the oracle's path,
    caches, and 32 greedy tokens after a 16-token prompt."""
    cfg = dict(synth.CONFIGS["gpt2-124m"])
    gpu, cpu, _ = gpt2_pair(cfg, seed=3, fused=fused, scale=0.0005)
    prompt = synth.prompt(16, cfg["n_vocab"], 3)
    compare_steps(gpu, cpu, prompt[:8], what="gpt2-124m")
    exp = cpu.decode(prompt, 32)
    got = gpu.decode(prompt, 32)
    assert np.array_equal(got, exp), f"first difference at {np.nonzero(got != exp)[0][:1]}"
