"""Temperature / top-p sampling on the device against the restatement of Sampler::sample
(crates/wgml/src/models/sampler.rs:32-131) fed the same uniform draws.

Token ids must be identical, draw by draw.  The device adds the softmax denominator and walks the CDF in the
reference's order, so the only licence left is the last bit of expf (CUDA's and the host's differ on some
arguments): a draw whose coin falls within 1e-5 of a CDF step or of the nucleus boundary (the oracle reports the
distance, relative to the probability mass walked) may land on a neighbouring token, and so may a draw that picks
among candidates whose probabilities agree to 2e-6 relative (their order in the sorted list is decided by that
last bit).  Such draws are counted and must be rare."""
import numpy as np
import pytest
import torch

import oracle
from helpers import SMALL_GPT2, SMALL_LLAMA, gpt2_pair, llama_pair
from wgml_b200 import ops, synth

pytestmark = pytest.mark.gpu


def _logit_sets(n):
    rng = np.random.default_rng(12)
    yield "peaked", (rng.standard_normal(n) * 6).astype(np.float32)
    yield "moderate", (rng.standard_normal(n) * 1.5).astype(np.float32)
    yield "flat", (rng.standard_normal(n) * 0.05).astype(np.float32)          # nearly every token in the nucleus
    ties = np.round(rng.standard_normal(n) * 2).astype(np.float32)             # many exactly equal probabilities
    yield "ties", ties
    big = (rng.standard_normal(n) * 300 + 1000).astype(np.float32)             # the scale random-weight models produce
    yield "huge", big


@pytest.mark.parametrize("n", [32000, 50257, 1000])
@pytest.mark.parametrize("temperature,topp", [(0.7, 0.95), (1.0, 0.5), (1.3, 1.0), (0.7, 0.0), (0.0, 0.9)])
def test_sample_matches_the_oracle_draw_by_draw(n, temperature, topp):
    draws, excused, total = 64, 0, 0
    s = ops.Sampler(n, temperature, topp)
    for name, logits in _logit_sets(n):
        d = torch.from_numpy(logits).cuda()
        for i in range(draws):
            coin = ops.sampler_coin(99, total)
            assert coin == oracle.sampler_coin(99, total) and 0.0 <= coin < 1.0
            exp, slack = oracle.sample(logits, temperature, topp, coin)
            got = s.sample(d, coin)
            total += 1
            if got != exp:
                z = logits.astype(np.float32) / np.float32(temperature) if temperature else logits
                tied = abs(float(np.exp(np.float64(z[got]) - np.float64(z[exp]))) - 1.0) < 2e-6
                assert slack < 1e-5 or tied, (f"{name} draw {i}: token {got} vs {exp} with the coin {slack:.3g} away from a "
                                              f"CDF step and logits {z[got]!r} / {z[exp]!r}")
                excused += 1
        assert torch.equal(d.cpu(), torch.from_numpy(logits)), "the logits were modified"
    assert total >= 256 and excused <= max(1, total // 100), f"{excused} of {total} draws fell on a rounding boundary"


def test_coin_is_uniform_and_counter_based():
    c = np.array([ops.sampler_coin(7, i) for i in range(20000)])
    assert 0.0 <= c.min() and c.max() < 1.0 and abs(c.mean() - 0.5) < 0.01 and abs(np.mean(c < 0.1) - 0.1) < 0.01
    assert ops.sampler_coin(7, 5) == ops.sampler_coin(7, 5) != ops.sampler_coin(8, 5)


@pytest.mark.parametrize("family", ["llama", "gpt2"])
def test_token_loop_with_sampler_stays_on_the_device(family):
    """decode() with a temperature / top-p 0.95 sampler (the chat loop's Sampler::new(vocab, 0.7, 0.95),
    crates/wgml-chat/src/sampler.rs:109-110; random weights give logits far from unit scale, so the temperature
    is set to their spread to keep the draws varied) against the oracle transformer + oracle sampler fed the
    loop's coins: same ids for 48 generated tokens, in one call and resumed half way."""
    if family == "llama":
        cfg = dict(SMALL_LLAMA)
        gpu, cpu, _ = llama_pair(cfg, seed=9, scale=0.0005)
        vocab = cfg["vocab_size"]
    else:
        cfg = dict(SMALL_GPT2)
        gpu, cpu, _ = gpt2_pair(cfg, seed=9, scale=0.002)
        vocab = cfg["n_vocab"]
    prompt = synth.prompt(5, vocab, 9)
    seed, n_gen = 1234, 48
    temp = float(np.float32(0.7 * np.std(cpu.forward(int(prompt[0]), 0))))
    exp, slacks, tok = [], [], int(prompt[0])
    for pos in range(len(prompt) - 1 + n_gen):
        logits = cpu.forward(tok, pos)
        if pos + 1 < len(prompt):
            tok = int(prompt[pos + 1])
            slacks.append(1.0)
        else:
            tok, sl = oracle.sample(logits, temp, 0.95, oracle.sampler_coin(seed, pos + 1))
            slacks.append(sl)
        exp.append(tok)
    exp = np.array(exp, np.uint32)
    gpu.set_sampler(temp, 0.95, seed)
    got = gpu.decode(prompt, n_gen)
    diff = np.nonzero(got != exp)[0]
    assert diff.size == 0 or slacks[diff[0]] < 1e-4, f"first difference at step {diff[0]} (slack {slacks[diff[0]]:.3g}): {got[diff[0]]} vs {exp[diff[0]]}"
    assert len(set(exp[len(prompt) - 1:].tolist())) > 4, "the draws should not collapse onto one token"
    if diff.size == 0:
        # resumable: the coin depends on the position only
        first = gpu.decode(prompt, 20)
        rest = gpu.decode(first[-1:], n_gen - 20, start_pos=len(first))
        assert np.array_equal(np.concatenate([first, rest]), exp)
    # back to greedy
    gpu.set_sampler(0.0, 0.0, 0)
    greedy = gpu.decode(prompt, 8)
    ref = cpu.decode(prompt, 8)
    ref = ref[0] if isinstance(ref, tuple) else ref
    assert np.array_equal(greedy, ref)
