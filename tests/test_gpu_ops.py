"""Stand-alone operators against their CPU twins in the oracle; sizes follow the reference's own
GPU-vs-CPU tests (n = 1757, head 128 with 13 / 9 heads at pos 10, ...)."""
import numpy as np
import pytest
import torch

import oracle
from conftest import assert_close
from wgml_b200 import ops

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


@pytest.mark.parametrize("n", [1, 7, 1757, 4096, 8192])
def test_rms_norm(n):  # ops/rms_norm.rs:77-136
    rng = np.random.default_rng(n)
    v, w = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    for eps in (1e-5, 1e-6):
        out = torch.zeros(n, device="cuda")
        ops.RmsNorm.from_device().dispatch(ops.RmsNormConfig(eps), out, dev(v), dev(w))
        assert_close(out.cpu().numpy(), oracle.rms_norm(v, w, eps), 1e-5, 1e-6, "rms_norm")


@pytest.mark.parametrize("n", [2, 768, 1757])
def test_layernorm(n):  # ops/layernorm.rs:67-102
    v = np.random.default_rng(n).standard_normal(n).astype(np.float32) * 3 + 1
    out = torch.zeros(n, device="cuda")
    ops.LayerNorm.from_device().dispatch(out, dev(v))
    assert_close(out.cpu().numpy(), oracle.layernorm(v), 1e-5, 1e-6, "layernorm")
    with pytest.raises(ops.WgbError):
        ops.LayerNorm.from_device().dispatch(torch.zeros(n + 1, device="cuda"), dev(v))


@pytest.mark.parametrize("variant", [ops.RoPEVariant.Original, ops.RoPEVariant.Neox])
@pytest.mark.parametrize("case", [(128, 13, 9, 10), (48, 6, 6, 255), (128, 64, 8, 4223), (64, 12, 12, 0)])
def test_rope(variant, case):  # ops/rope.rs:131-198
    hs, nq, nk, pos = case
    rng = np.random.default_rng(hs + pos)
    q, k = rng.standard_normal(nq * hs).astype(np.float32), rng.standard_normal(nk * hs).astype(np.float32)
    qd, kd = dev(q), dev(k)
    cfg = ops.RoPEConfig(hs, nk * hs, pos, 10000.0)
    ops.RoPE.from_device().dispatch(variant, cfg, qd, kd)
    qe, ke = oracle.rope(int(variant), q, k, hs, nk * hs, pos)
    assert_close(qd.cpu().numpy(), qe, 1e-5, 1e-5, "rope q")
    assert_close(kd.cpu().numpy(), ke, 1e-5, 1e-5, "rope k")


def test_rope_argument_checks():  # ops/rope.rs:51-56
    r = ops.RoPE.from_device()
    cfg = ops.RoPEConfig(4, 4, 1, 10000.0)
    with pytest.raises(ops.WgbError):
        r.dispatch(0, cfg, torch.zeros(7, device="cuda"), torch.zeros(4, device="cuda"))
    with pytest.raises(ops.WgbError) as e:
        r.dispatch(0, cfg, torch.zeros(4, device="cuda"), torch.zeros(8, device="cuda"))
    assert "Query vector" in str(e.value)


def test_softmax_columns():  # ops/softmax.rs:63-95
    rng = np.random.default_rng(9)
    nrows, ncols, stride = 1757, 5, 1760
    m = rng.standard_normal(ncols * stride).astype(np.float32) * 4
    d = dev(m)
    ops.SoftMax.from_device().dispatch(d, nrows, ncols, stride)
    got = d.cpu().numpy()
    for j in range(ncols):
        assert_close(got[j * stride:j * stride + nrows], oracle.softmax(m[j * stride:j * stride + nrows]), 1e-5, 1e-7, "softmax")
        assert np.array_equal(got[j * stride + nrows:(j + 1) * stride], m[j * stride + nrows:(j + 1) * stride])  # padding untouched


def test_silu():  # ops/silu.rs:57-98
    rng = np.random.default_rng(10)
    a, b = rng.standard_normal(1757).astype(np.float32) * 3, rng.standard_normal(1757).astype(np.float32)
    d = dev(a)
    ops.Silu.from_device().dispatch(d, dev(b))
    assert_close(d.cpu().numpy(), oracle.silu(a, b), 1e-5, 1e-6, "silu")


@pytest.mark.parametrize("op", list(ops.UnaryOp))
def test_unary(op):  # ops/unary.rs:273-348
    rng = np.random.default_rng(int(op))
    v = rng.standard_normal(1757).astype(np.float32) * 2
    if op in (ops.UnaryOp.Sqrt, ops.UnaryOp.Log):
        v = np.abs(v) + 0.01
    args = (0.3, 0.9) if op.has_args() else None
    exp = oracle.unary(int(op), v, (0.3, 0.9, 0, 0))
    dst = torch.zeros(1757, device="cuda")
    ops.Unary(None, op).dispatch(dst, dev(v), args)
    assert_close(dst.cpu().numpy(), exp, 1e-5, 1e-6, op.name)
    src = dev(v)
    ops.UnaryInplace(None, op).dispatch(src, args)
    assert_close(src.cpu().numpy(), exp, 1e-5, 1e-6, op.name + " in place")
    with pytest.raises(ops.WgbError):  # "Unary ops argument mismatch."
        ops.Unary(None, op).dispatch(dst, dev(v), None if op.has_args() else (1.0,))


def test_op_assign():
    rng = np.random.default_rng(12)
    a, b = rng.standard_normal(1000).astype(np.float32), rng.standard_normal(1000).astype(np.float32)
    for kind, exp in ((ops.OpAssignVariant.Add, a + b), (ops.OpAssignVariant.Mul, a * b), (ops.OpAssignVariant.Copy, b)):
        d = dev(a)
        ops.OpAssign(None, kind).dispatch(d, dev(b))
        assert np.array_equal(d.cpu().numpy(), exp)
    # contiguous sub-views: rows(768, 768) of a 2304-vector
    big = dev(np.arange(2304))
    dst = torch.zeros(768, device="cuda")
    ops.OpAssign(None, ops.OpAssignVariant.Copy).dispatch(dst, big[768:1536])
    assert np.array_equal(dst.cpu().numpy(), np.arange(768, 1536, dtype=np.float32))


def test_argmax_first_maximum():
    v = np.random.default_rng(13).standard_normal(50257).astype(np.float32)
    assert ops.sample_argmax(dev(v)) == oracle.argmax(v) == int(np.argmax(v))
    v[[40000, 123, 999]] = v.max() + 1  # ties: the lowest index wins, as nalgebra's imax
    assert ops.sample_argmax(dev(v)) == 123
    assert ops.sample_argmax(dev(np.array([-3.0], np.float32))) == 0
    assert ops.sample_argmax(dev(-np.arange(1, 70000))) == 0
