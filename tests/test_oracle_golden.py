"""Pins the CPU oracle: dequantisation against the reference test's block patterns (expected values
from gguf-py, see tests/golden/make_golden.py), f16 decoding against every bit pattern, and the
small ops against independent numpy formulas."""
import numpy as np
import pytest

import oracle
from conftest import assert_bit_exact, assert_close

QTYPES = [oracle.Q4_0, oracle.Q4_1, oracle.Q5_0, oracle.Q5_1, oracle.Q8_0, oracle.Q4_K, oracle.Q5_K, oracle.Q6_K, oracle.Q8_K]


@pytest.mark.parametrize("qtype", QTYPES)
@pytest.mark.parametrize("kind", ["pattern", "random"])
def test_dequantize_matches_golden(golden, qtype, kind):
    got = oracle.dequantize(qtype, golden[f"{kind}_in_{qtype}"])
    assert_bit_exact(got, golden[f"{kind}_out_{qtype}"], f"{kind} {oracle.QTYPE_NAMES[qtype]}")


def test_decode_f16_all_bit_patterns(golden):
    exp = golden["f16_all"]
    got = np.array([oracle.decode_f16(i) for i in range(65536)], dtype=np.float32)
    nan = np.isnan(exp)
    assert np.array_equal(np.isnan(got), nan)
    assert_bit_exact(got[~nan], exp[~nan], "f16")
    # f32::NAN, negated when the sign bit is set (quantization.rs:402-408)
    assert got[0x7e00:0x7e01].view(np.uint32)[0] == 0x7FC00000
    assert got[0xfe00:0xfe01].view(np.uint32)[0] == 0xFFC00000


def test_gemv_quant_is_dequantize_then_dot(golden):
    rng = np.random.default_rng(1)
    for qtype in (oracle.Q8_0, oracle.Q4_K, oracle.Q6_K):
        bl = oracle.BLOCK_LEN[qtype]
        raw = golden[f"random_in_{qtype}"]
        nblocks = raw.size // oracle.BLOCK_BYTES[qtype]
        nrows = 4
        ncols = nblocks // nrows * bl
        raw = raw[: nrows * (ncols // bl) * oracle.BLOCK_BYTES[qtype]]
        x = rng.standard_normal(ncols).astype(np.float32)
        w = oracle.dequantize(qtype, raw).reshape(nrows, ncols)
        out, out64 = oracle.gemv_quant(qtype, raw, nrows, ncols, x, want_f64=True)
        assert_close(out64, w.astype(np.float64) @ x.astype(np.float64), rtol=1e-12, atol=1e-12, what="f64 gemv")
        assert_close(out, out64, rtol=1e-4, atol=1e-4, what="f32 gemv")


def test_small_ops_against_numpy():
    rng = np.random.default_rng(2)
    v = rng.standard_normal(1757).astype(np.float32)
    w = rng.standard_normal(1757).astype(np.float32)
    rms = 1.0 / np.sqrt((v.astype(np.float64) ** 2).mean() + 1e-5)
    assert_close(oracle.rms_norm(v, w, 1e-5), v * rms * w, rtol=1e-5, atol=1e-6, what="rms_norm")
    ln = (v - v.mean(dtype=np.float64)) / np.sqrt(v.astype(np.float64).var() + 1e-5)
    assert_close(oracle.layernorm(v), ln, rtol=1e-5, atol=1e-6, what="layernorm")
    e = np.exp(v.astype(np.float64) - v.max())
    assert_close(oracle.softmax(v), e / e.sum(), rtol=1e-5, atol=1e-9, what="softmax")
    assert_close(oracle.silu(v, w), w * (v / (1 + np.exp(-v.astype(np.float64)))), rtol=1e-5, atol=1e-6, what="silu")
    assert oracle.argmax(np.array([1, 5, 5, 2], np.float32)) == 1  # first maximum


def test_rope_variants():
    rng = np.random.default_rng(3)
    hs, nq, nk, pos = 128, 13, 9, 10  # the sizes of the reference's gpu_rope test (ops/rope.rs:131-198)
    q = rng.standard_normal(nq * hs).astype(np.float32)
    k = rng.standard_normal(nk * hs).astype(np.float32)
    q0, k0 = oracle.rope(0, q, k, hs, nk * hs, pos)
    i = np.arange(0, hs, 2)
    ang = pos * (10000.0 ** (-(i / hs)))
    c, s = np.cos(ang), np.sin(ang)
    qe = q.reshape(nq, hs // 2, 2).astype(np.float64)
    exp = np.stack([c * qe[..., 0] - s * qe[..., 1], s * qe[..., 0] + c * qe[..., 1]], -1).reshape(-1)
    assert_close(q0, exp, rtol=1e-4, atol=1e-5, what="rope original q")
    assert not np.allclose(k0, k)
    # Neox: pairs (j, j + hs/2) inside every head
    q1, _ = oracle.rope(1, q, k, hs, nk * hs, pos)
    qn = q.reshape(nq, 2, hs // 2).astype(np.float64)
    exp = np.stack([c * qn[:, 0] - s * qn[:, 1], s * qn[:, 0] + c * qn[:, 1]], 1).reshape(-1)
    assert_close(q1, exp, rtol=1e-4, atol=1e-5, what="rope neox q")


def test_attention_against_numpy():
    rng = np.random.default_rng(4)
    seq_len, n_heads, hs, kv_mul, pos = 64, 12, 16, 3, 37
    kv_dim = n_heads // kv_mul * hs
    q = rng.standard_normal(n_heads * hs).astype(np.float32)
    kc = rng.standard_normal((seq_len, kv_dim)).astype(np.float32)
    vc = rng.standard_normal((seq_len, kv_dim)).astype(np.float32)
    xb, attn = oracle.attention(seq_len, kv_dim, kv_mul, n_heads, hs, pos, q, kc, vc)
    for h in range(n_heads):
        kh = kc[: pos + 1, (h // kv_mul) * hs:(h // kv_mul + 1) * hs].astype(np.float64)
        vh = vc[: pos + 1, (h // kv_mul) * hs:(h // kv_mul + 1) * hs].astype(np.float64)
        s = kh @ q[h * hs:(h + 1) * hs] / np.sqrt(hs)
        p = np.exp(s - s.max())
        p /= p.sum()
        assert_close(attn[h, : pos + 1], p, rtol=1e-4, atol=1e-6, what="attn weights")
        assert_close(xb[h * hs:(h + 1) * hs], p @ vh, rtol=1e-4, atol=1e-5, what="attn out")


def test_unary_ops_known_values():
    x = np.array([-2.0, -0.5, 0.0, 0.5, 3.0], np.float32)
    assert np.array_equal(oracle.unary(oracle.UNARY_OPS.index("Relu"), x), np.maximum(x, 0))
    assert np.array_equal(oracle.unary(oracle.UNARY_OPS.index("Sgn"), x), np.array([-1, -1, 1, 1, 1], np.float32))
    assert np.array_equal(oracle.unary(oracle.UNARY_OPS.index("Clamp"), x, (-1.0, 1.0, 0, 0)), np.clip(x, -1, 1))
    g = oracle.unary(oracle.UNARY_OPS.index("Gelu"), x)
    exp = 0.5 * x * (1 + np.tanh(0.7978846 * x * (1 + 0.044715 * x * x)))
    assert_close(g, exp, rtol=1e-5, atol=1e-6, what="gelu")
