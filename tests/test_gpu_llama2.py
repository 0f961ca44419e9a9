"""Llama-2 forward and token loop against the CPU transformer (oracle).

Logits are compared step by step with the oracle fed the same tokens: within 1e-3 relative / 1e-4
absolute, the absolute term scaled by the largest logit magnitude (random-weight models produce
logits far from unit scale).  Greedy tokens must be identical for the first 32 generated steps."""
import numpy as np
import pytest
import torch

import oracle
from conftest import ATOL, RTOL, assert_close
from helpers import SMALL_LLAMA, llama_pair, rel_err
from wgml_b200 import synth
from wgml_b200.gguf import Gguf
from wgml_b200.models import Llama2, LlamaModelType

pytestmark = pytest.mark.gpu


def compare_steps(gpu, cpu, tokens, start=0, what=""):
    for i, tok in enumerate(tokens):
        gpu.dispatch(int(tok), start + i)
        got = gpu.logits().cpu().numpy()
        exp = cpu.forward(int(tok), start + i)
        scale = max(1.0, float(np.abs(exp).max()))
        assert_close(got, exp, RTOL, ATOL * scale, f"{what} logits at step {i}")
    kc, vc = cpu.caches()
    for l in range(gpu.config.n_layers):
        n = start + len(tokens)
        s = max(1.0, float(np.abs(kc[l, :n]).max()))
        assert_close(gpu.key_cache(l)[:n].cpu().numpy(), kc[l, :n], RTOL, ATOL * s, f"{what} key cache {l}")
        s = max(1.0, float(np.abs(vc[l, :n]).max()))
        assert_close(gpu.value_cache(l)[:n].cpu().numpy(), vc[l, :n], RTOL, ATOL * s, f"{what} value cache {l}")


@pytest.mark.parametrize("fused", [True, False])
def test_tiny_llama_f32_logits_and_greedy_tokens(fused):
    """Tiny Llama-2 (dim 288, 6 layers, head 48, vocab 32000, f32): 8 prompt ids, 128 greedy steps."""
    cfg = synth.CONFIGS["tiny-llama"]
    gpu, cpu, _ = llama_pair(cfg, seed=1, fused=fused)
    prompt = synth.prompt(8, cfg["vocab_size"], seed=1)
    exp_tokens, margin = cpu.decode(prompt, 128)
    got_tokens = gpu.decode(prompt, 128)
    assert np.array_equal(got_tokens[:7], prompt[1:])  # forced prompt tokens
    assert np.array_equal(got_tokens[: 7 + 32], exp_tokens[: 7 + 32]), "greedy tokens differ within the first 32 steps"
    first_diff = np.nonzero(got_tokens != exp_tokens)[0]
    if first_diff.size:  # later divergence is only acceptable at a numerical tie
        assert margin[first_diff[0]] < 1e-3 * 10, f"diverged at step {first_diff[0]} with top-2 margin {margin[first_diff[0]]}"
    # logits along the oracle's own token path
    gpu2, cpu2, _ = llama_pair(cfg, seed=1, fused=fused)
    path = np.concatenate([prompt[:1], exp_tokens[:15]])
    compare_steps(gpu2, cpu2, path, what="tiny")


@pytest.mark.parametrize("qtype", [synth.Q4_K, synth.Q6_K, synth.Q8_0, synth.Q5_K, synth.Q4_0])
@pytest.mark.parametrize("fused", [True, False])
def test_small_quantised_llama(qtype, fused):
    cfg = dict(SMALL_LLAMA, default_qtype=qtype)
    gpu, cpu, _ = llama_pair(cfg, seed=2, fused=fused, scale=0.002)
    compare_steps(gpu, cpu, synth.prompt(12, cfg["vocab_size"], 2), what=f"qtype {qtype}")


def test_mixed_formats_in_one_layer_fall_back_to_separate_launches():
    cfg = dict(SMALL_LLAMA)
    t = synth.llama_tensors(cfg, 3, scale=0.002)
    t["blk.0.attn_v.weight"] = synth.matrix(synth.Q6_K, 512, 512, 3, "v6", 0.002)
    t["blk.1.ffn_up.weight"] = synth.matrix(synth.Q8_0, 1024, 512, 3, "up8", 0.002)
    gpu, cpu, _ = llama_pair(cfg, tensors=t)
    compare_steps(gpu, cpu, synth.prompt(6, cfg["vocab_size"], 3), what="mixed")


@pytest.mark.parametrize("fused", [True, False])
def test_qwen2_variant_gqa_bias_neox(fused):
    """Qwen2 = biases on q/k/v + Neox RoPE (models/llama2/mod.rs:27-32), with grouped-query heads."""
    cfg = dict(SMALL_LLAMA, n_kv_heads=2, default_qtype=synth.Q4_K)
    gpu, cpu, _ = llama_pair(cfg, seed=4, biases=True, qwen=True, scale=0.002, fused=fused)
    compare_steps(gpu, cpu, synth.prompt(10, cfg["vocab_size"], 4), what="qwen2")


def test_7b_shapes_two_layers_q4_k_m_mix():
    """Llama-2-7B dimensions (dim 4096, 32 heads x 128, FFN 11008, vocab 32000, Q4_K + Q6_K mix) with
    2 layers so that the CPU oracle finishes in seconds."""
    cfg = dict(synth.CONFIGS["llama2-7b"], n_layers=2, seq_len=64)
    gpu, cpu, _ = llama_pair(cfg, seed=5, scale=0.0005)
    prompt = synth.prompt(4, cfg["vocab_size"], 5)
    compare_steps(gpu, cpu, prompt, what="7b-2l")
    exp, _ = cpu.decode(prompt, 8, 0)
    assert np.array_equal(gpu.decode(prompt, 8), exp)


def test_decode_is_deterministic_and_resumable():
    cfg = dict(SMALL_LLAMA)
    gpu, cpu, _ = llama_pair(cfg, seed=6, scale=0.002)
    prompt = synth.prompt(5, cfg["vocab_size"], 6)
    a = gpu.decode(prompt, 20)
    b = gpu.decode(prompt, 20)
    assert np.array_equal(a, b)
    # resume at start_pos with the cache left by the first call (chat_llama2.rs:57,98)
    first = gpu.decode(prompt, 6)
    rest = gpu.decode(first[-1:], 14, start_pos=len(first))
    assert np.array_equal(np.concatenate([first, rest]), a)
    exp, _ = cpu.decode(prompt, 20)
    assert np.array_equal(a, exp)


def test_argument_errors():
    cfg = dict(SMALL_LLAMA)
    gpu, _, t = llama_pair(cfg, seed=7)
    with pytest.raises(Exception):
        gpu.dispatch(cfg["vocab_size"], 0)
    with pytest.raises(Exception):
        gpu.dispatch(0, cfg["seq_len"])
    with pytest.raises(Exception):
        gpu.decode(np.array([1, 2], np.uint32), cfg["seq_len"])
    empty = Llama2(gpu.config)
    with pytest.raises(Exception) as e:
        empty.dispatch(0, 0)
    assert "never set" in str(e.value)


def test_load_from_gguf_file(tmp_path):
    """Llama2Weights::from_gguf path: a GGUF written with gguf-py (quantised tensors) -> device -> logits."""
    import gguf
    cfg = dict(SMALL_LLAMA, n_kv_heads=4)
    t = synth.llama_tensors(cfg, 8, scale=0.002)
    path = str(tmp_path / "small.gguf")
    w = gguf.GGUFWriter(path, "llama")
    w.add_uint32("llama.embedding_length", cfg["dim"])
    w.add_uint32("llama.feed_forward_length", cfg["hidden_dim"])
    w.add_uint32("llama.block_count", cfg["n_layers"])
    w.add_uint32("llama.attention.head_count", cfg["n_q_heads"])
    w.add_uint32("llama.attention.head_count_kv", cfg["n_kv_heads"])
    w.add_uint32("llama.context_length", cfg["seq_len"])
    w.add_float32("llama.attention.layer_norm_rms_epsilon", 1e-5)
    w.add_array("tokenizer.ggml.tokens", [f"t{i}" for i in range(cfg["vocab_size"])])
    shapes = {"attn_q": (512, 512), "attn_k": (256, 512), "attn_v": (256, 512), "attn_output": (512, 512),
              "ffn_gate": (1024, 512), "ffn_up": (1024, 512), "ffn_down": (512, 1024), "token_embd": (1000, 512), "output": (1000, 512)}
    for name, (qt, arr) in t.items():
        base = name.split(".")[-2]
        if qt == synth.F32:
            w.add_tensor(name, np.asarray(arr, np.float32))
        else:
            r, c = shapes[base]
            w.add_tensor(name, np.asarray(arr).reshape(r, c // 256 * 144), raw_dtype=gguf.GGMLQuantizationType.Q4_K)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    g = Gguf.open(path)
    gpu = Llama2.from_gguf(g, LlamaModelType.Llama)
    assert gpu.config.vocab_size == 1000 and gpu.config.n_kv_heads == 4 and abs(gpu.config.rms_norm_eps - 1e-5) < 1e-9
    nbytes, secs = gpu.load_stats()   # the pipelined upload moved every matrix once
    assert nbytes == sum(np.asarray(a).nbytes for n_, (q_, a) in t.items() if n_.endswith(".weight") and "norm" not in n_) and secs > 0
    cpu = oracle.Llama2Oracle(cfg, t)
    compare_steps(gpu, cpu, synth.prompt(5, 1000, 8), what="gguf")


def test_llama2_7b_full_depth_greedy_tokens():
    """The whole Llama-2-7B configuration (32 layers, Q4_K with Q6_K for the output matrix and every other
    ffn_down) against the CPU transformer with on-the-fly dequantisation: logits at the first steps and the
    first 32 greedy tokens after a 4-token prompt.  Weight scales are chosen so that pre-activations stay of
    order one; at the scale of the timing configuration a random 32-layer network amplifies f32 rounding
    differences until implementations cannot be compared token by token."""
    cfg = dict(synth.CONFIGS["llama2-7b"], seq_len=48)
    gpu, cpu, _ = llama_pair(cfg, seed=4, scale=1.0e-4)
    prompt = synth.prompt(4, cfg["vocab_size"], 4)
    exp_tokens, margin = cpu.decode(prompt, 32)
    got_tokens = gpu.decode(prompt, 32)
    diff = np.nonzero(got_tokens != exp_tokens)[0]
    assert diff.size == 0, f"first difference at step {diff[0]}, top-2 margin there {margin[diff[0]]}"
    gpu2, cpu2, _ = llama_pair(cfg, seed=4, scale=1.0e-4)
    compare_steps(gpu2, cpu2, np.concatenate([prompt[:1], exp_tokens[:3]]), what="7b")


def test_70b_shapes_two_layers_gqa():
    """Llama-2-70B dimensions (dim 8192, 64 query / 8 KV heads of 128, FFN 28672, vocab 32000, Q4_K) with 2
    layers: the long rows (K = 8192 and 28672) and the grouped-query attention path at the real sizes."""
    cfg = dict(synth.CONFIGS["llama2-70b"], n_layers=2, seq_len=48)
    gpu, cpu, _ = llama_pair(cfg, seed=6, scale=2.0e-4)
    prompt = synth.prompt(4, cfg["vocab_size"], 6)
    compare_steps(gpu, cpu, prompt, what="70b-2l")
    exp, _ = cpu.decode(prompt, 8, 0)
    assert np.array_equal(gpu.decode(prompt, 8), exp)
