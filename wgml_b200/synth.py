"""Seeded synthetic weights for the benchmark and parity configurations.

No model file exists offline, so every configuration is filled with random blocks of the stated
distributions: quant codes uniform, f16 block scales = f16(|N(0,1)| * 0.01), f32 matrices
~N(0, 0.02), norm gains 1 + N(0, 0.02), biases ~N(0, 0.02).  The generator is numpy's PCG64 keyed by
(seed, tensor name), so the CPU oracle and the CUDA side rebuild identical bytes independently.
"""
from __future__ import annotations

import zlib

import numpy as np

F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q4_K, Q5_K, Q6_K, Q8_K = 0, 1, 2, 3, 6, 7, 8, 12, 13, 14, 15
BLOCK_BYTES = {F32: 4, F16: 2, Q4_0: 18, Q4_1: 20, Q5_0: 22, Q5_1: 24, Q8_0: 34, Q4_K: 144, Q5_K: 176, Q6_K: 210, Q8_K: 292}
BLOCK_LEN = {F32: 1, F16: 1, Q4_0: 32, Q4_1: 32, Q5_0: 32, Q5_1: 32, Q8_0: 32, Q4_K: 256, Q5_K: 256, Q6_K: 256, Q8_K: 256}
# byte offsets of the f16 scale fields inside a block
_F16_SCALES = {Q4_0: (0,), Q5_0: (0,), Q8_0: (0,), Q4_1: (0, 2), Q5_1: (0, 2), Q4_K: (0, 2), Q5_K: (0, 2), Q6_K: (208,)}

CONFIGS = {
    # tiny Llama-2 architecture, f32 weights
    "tiny-llama": dict(arch="llama", dim=288, hidden_dim=768, n_layers=6, n_q_heads=6, n_kv_heads=6, vocab_size=32000,
                       seq_len=256, rope_base_freq=10000.0, rms_norm_eps=1e-5, default_qtype=F32),
    # Llama-2-7B architecture, Q4_K_M-style mix
    "llama2-7b": dict(arch="llama", dim=4096, hidden_dim=11008, n_layers=32, n_q_heads=32, n_kv_heads=32, vocab_size=32000,
                      seq_len=768, rope_base_freq=10000.0, rms_norm_eps=1e-5, default_qtype=Q4_K, mix="q4_k_m"),
    # Llama-2-70B architecture, all Q4_K
    "llama2-70b": dict(arch="llama", dim=8192, hidden_dim=28672, n_layers=80, n_q_heads=64, n_kv_heads=8, vocab_size=32000,
                       seq_len=4224, rope_base_freq=10000.0, rms_norm_eps=1e-5, default_qtype=Q4_K),
    # GPT-2 124M, Q8_0 matrices
    "gpt2-124m": dict(arch="gpt2", n_vocab=50257, n_seq=1024, n_embd=768, n_head=12, n_layer=12, ff_len=3072,
                      default_qtype=Q8_0),
}


def _rng(seed: int, name: str) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64([seed, zlib.crc32(name.encode())]))


def quant_blocks(qtype: int, nblocks: int, rng: np.random.Generator, scale: float = 0.01) -> np.ndarray:
    """`nblocks` raw GGUF blocks as a flat uint8 array."""
    bb = BLOCK_BYTES[qtype]
    nbytes = nblocks * bb
    raw = rng.integers(0, 1 << 63, size=(nbytes + 7) // 8, dtype=np.int64).view(np.uint8)[:nbytes].copy()
    # the top bit of every int64 is never set above: redraw those bytes so all 256 values occur
    raw[7::8] = rng.integers(0, 256, size=raw[7::8].size, dtype=np.uint8)
    blocks = raw.reshape(nblocks, bb)
    for off in _F16_SCALES.get(qtype, ()):
        s = (np.abs(rng.standard_normal(nblocks, dtype=np.float32)) * np.float32(scale)).astype(np.float16)
        blocks[:, off:off + 2] = s.view(np.uint8).reshape(nblocks, 2)
    if qtype == Q8_K:
        s = np.abs(rng.standard_normal(nblocks, dtype=np.float32)) * np.float32(scale)
        blocks[:, 0:4] = s.view(np.uint8).reshape(nblocks, 4)
    return raw


def matrix(qtype: int, nrows: int, ncols: int, seed: int, name: str, scale: float = 0.01):
    """(qtype, array) for an nrows x ncols matrix: raw blocks (uint8) or f32 values."""
    rng = _rng(seed, name)
    if qtype == F32:
        return F32, (rng.standard_normal(nrows * ncols, dtype=np.float32) * np.float32(0.02))
    if qtype == F16:
        return F16, (rng.standard_normal(nrows * ncols, dtype=np.float32) * np.float32(0.02)).astype(np.float16).view(np.uint8)
    assert ncols % BLOCK_LEN[qtype] == 0
    return qtype, quant_blocks(qtype, nrows * (ncols // BLOCK_LEN[qtype]), rng, scale)


def vector(n: int, seed: int, name: str, mean: float = 0.0) -> tuple:
    rng = _rng(seed, name)
    return F32, (np.float32(mean) + rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)).astype(np.float32)


def llama_tensors(cfg: dict, seed: int = 0, biases: bool = False, scale: float = 0.01, layers=None,
                  model_tensors: bool = True) -> dict:
    """All tensors of a Llama-architecture model, GGUF names -> (qtype, array).  `layers` restricts the
    blocks generated; `model_tensors=False` leaves out token_embd / output / output_norm."""
    dim, hid, vocab = cfg["dim"], cfg["hidden_dim"], cfg["vocab_size"]
    kv_dim = dim * cfg["n_kv_heads"] // cfg["n_q_heads"]
    qt = cfg.get("default_qtype", Q4_K)
    mix = cfg.get("mix")
    t = {}
    for l in (range(cfg["n_layers"]) if layers is None else layers):
        p = f"blk.{l}."
        shapes = {"attn_q": (dim, dim), "attn_k": (kv_dim, dim), "attn_v": (kv_dim, dim), "attn_output": (dim, dim),
                  "ffn_gate": (hid, dim), "ffn_up": (hid, dim), "ffn_down": (dim, hid)}
        for nm, (r, c) in shapes.items():
            q = qt
            if mix == "q4_k_m" and nm == "ffn_down" and l % 2 == 0:
                q = Q6_K
            t[p + nm + ".weight"] = matrix(q, r, c, seed, p + nm, scale)
        t[p + "attn_norm.weight"] = vector(dim, seed, p + "attn_norm", 1.0)
        t[p + "ffn_norm.weight"] = vector(dim, seed, p + "ffn_norm", 1.0)
        if biases:
            t[p + "attn_q.bias"] = vector(dim, seed, p + "attn_q.bias")
            t[p + "attn_k.bias"] = vector(kv_dim, seed, p + "attn_k.bias")
            t[p + "attn_v.bias"] = vector(kv_dim, seed, p + "attn_v.bias")
    if model_tensors:
        t["token_embd.weight"] = matrix(qt, vocab, dim, seed, "token_embd", scale)
        t["output.weight"] = matrix(Q6_K if mix == "q4_k_m" else qt, vocab, dim, seed, "output", scale)
        t["output_norm.weight"] = vector(dim, seed, "output_norm", 1.0)
    return t


def gpt2_tensors(cfg: dict, seed: int = 0, scale: float = 0.01) -> dict:
    n, ff, vocab, nseq = cfg["n_embd"], cfg["ff_len"], cfg["n_vocab"], cfg["n_seq"]
    qt = cfg.get("default_qtype", Q8_0)
    t = {}
    for l in range(cfg["n_layer"]):
        p = f"blk.{l}."
        for nm, (r, c) in {"attn_qkv": (3 * n, n), "attn_output": (n, n), "ffn_up": (ff, n), "ffn_down": (n, ff)}.items():
            t[p + nm + ".weight"] = matrix(qt, r, c, seed, p + nm, scale)
            t[p + nm + ".bias"] = vector(r, seed, p + nm + ".bias")
        for nm in ("attn_norm", "ffn_norm"):
            t[p + nm + ".weight"] = vector(n, seed, p + nm + ".w", 1.0)
            t[p + nm + ".bias"] = vector(n, seed, p + nm + ".b")
    t["token_embd.weight"] = matrix(qt, vocab, n, seed, "token_embd", scale)
    t["position_embd.weight"] = matrix(F32, nseq, n, seed, "position_embd")
    t["output_norm.weight"] = vector(n, seed, "output_norm.w", 1.0)
    t["output_norm.bias"] = vector(n, seed, "output_norm.b")
    return t


def prompt(n: int, vocab: int, seed: int = 0) -> np.ndarray:
    return _rng(seed, "prompt").integers(0, vocab, size=n, dtype=np.uint32)


def model_bytes(tensors: dict) -> int:
    return int(sum(np.asarray(a).nbytes for _, a in tensors.values()))
