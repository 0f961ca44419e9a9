"""GemvQuant parity: CUDA (through the C ABI) against the oracle's dequantise-then-dot.

Tolerance: 1e-3 relative / 1e-4 absolute against the oracle's double-precision accumulation of the
same bit-exact weights, the absolute term in units of the output vector's RMS (the synthetic block
scales give outputs of order 1e2..1e3, where 1e-4 in absolute terms is below what any f32 summation
order can resolve).  The oracle's f32 result (sequential summation, as nalgebra does) carries its own
rounding error of up to about K * 2^-24 * sum|w x|, so against it the absolute term is widened by
that bound."""
import numpy as np
import pytest
import torch

import oracle
from conftest import ATOL, RTOL, assert_close
from wgml_b200 import ops, synth

pytestmark = pytest.mark.gpu
ALL = [ops.F32, ops.F16, ops.Q4_0, ops.Q4_1, ops.Q5_0, ops.Q5_1, ops.Q8_0, ops.Q4_K, ops.Q5_K, ops.Q6_K, ops.Q8_K]


def make(qtype, nrows, ncols, seed):
    qt, arr = synth.matrix(qtype, nrows, ncols, seed, f"m{qtype}")
    x = np.random.default_rng(seed + 1).standard_normal(ncols).astype(np.float32)
    return np.ascontiguousarray(arr).view(np.uint8), x


def check(qtype, raw, nrows, ncols, x, out):
    o32, o64 = oracle.gemv_quant(qtype, raw, nrows, ncols, x, want_f64=True)
    atol = ATOL * max(1.0, float(np.sqrt(np.mean(o64 ** 2))))
    assert_close(out, o64, RTOL, atol, f"qtype {qtype} {nrows}x{ncols} vs f64 oracle")
    w = oracle.dequantize(qtype, raw).reshape(nrows, ncols)
    bound = ncols * 2.0 ** -24 * (np.abs(w.astype(np.float64)) @ np.abs(x.astype(np.float64)))
    err = np.abs(out.astype(np.float64) - o32)
    assert (err <= atol + RTOL * np.abs(o32) + bound).all(), f"qtype {qtype}: vs f32 oracle, worst {err.max()}"


@pytest.mark.parametrize("qtype", ALL)
@pytest.mark.parametrize("shape", [(4, 256), (37, 512), (1757, 768), (1024, 2816)])
def test_gemv_small(qtype, shape):
    nrows, ncols = shape
    raw, x = make(qtype, nrows, ncols, 7)
    m = ops.GpuQuantMatrix(qtype, raw, nrows, ncols)
    out = torch.full((nrows,), float("nan"), device="cuda")
    ops.GemvQuant.from_device().dispatch(out, m, torch.from_numpy(x).cuda())
    check(qtype, raw, nrows, ncols, x, out.cpu().numpy())


@pytest.mark.parametrize("qtype", [ops.Q4_K, ops.Q8_0, ops.Q6_K, ops.Q5_0, ops.F32])
def test_gemv_raw_blocks_on_device(qtype):
    nrows, ncols = 130, 1024
    raw, x = make(qtype, nrows, ncols, 11)
    out = torch.zeros(nrows, device="cuda")
    ops.GemvQuant.from_device().dispatch_raw(out, qtype, torch.from_numpy(raw).cuda(), nrows, ncols, torch.from_numpy(x).cuda())
    check(qtype, raw, nrows, ncols, x, out.cpu().numpy())


@pytest.mark.parametrize("qtype", [ops.Q8_0, ops.Q4_K, ops.Q6_K])
@pytest.mark.parametrize("shape", [(4096, 4096), (11008, 4096), (4096, 11008), (32000, 4096)])
def test_gemv_microbench_shapes_vs_oracle(qtype, shape):
    """The GEMV microbench configurations at full size."""
    nrows, ncols = shape
    raw, x = make(qtype, nrows, ncols, 13)
    m = ops.GpuQuantMatrix(qtype, raw, nrows, ncols)
    out = torch.zeros(nrows, device="cuda")
    g = ops.GemvQuant.from_device()
    xd = torch.from_numpy(x).cuda()
    g.dispatch(out, m, xd)
    o = out.cpu().numpy()
    check(qtype, raw, nrows, ncols, x, o)
    # linearity: W(2x - 3y) = 2Wx - 3Wy (size-independent property)
    y = torch.randn(ncols, device="cuda", generator=torch.Generator("cuda").manual_seed(3))
    out_y, out_c = torch.zeros_like(out), torch.zeros_like(out)
    g.dispatch(out_y, m, y)
    g.dispatch(out_c, m, (2 * xd - 3 * y).contiguous())
    lin = (2 * out - 3 * out_y).cpu().numpy()
    scale = float(np.abs(lin).max())
    assert np.abs(out_c.cpu().numpy() - lin).max() <= 1e-5 * scale


def test_gemv_70b_and_gpt2_shapes():
    for qtype, (nrows, ncols) in [(ops.Q4_K, (1024, 8192)), (ops.Q4_K, (8192, 28672)), (ops.Q8_0, (2304, 768)),
                                  (ops.Q8_0, (50257, 768)), (ops.Q8_0, (768, 3072))]:
        raw, x = make(qtype, nrows, ncols, 17)
        m = ops.GpuQuantMatrix(qtype, raw, nrows, ncols)
        out = torch.zeros(nrows, device="cuda")
        ops.GemvQuant.from_device().dispatch(out, m, torch.from_numpy(x).cuda())
        check(qtype, raw, nrows, ncols, x, out.cpu().numpy())


def test_gemv_dimension_mismatch_is_an_error():
    raw, x = make(ops.Q4_K, 8, 256, 1)
    m = ops.GpuQuantMatrix(ops.Q4_K, raw, 8, 256)
    g = ops.GemvQuant.from_device()
    with pytest.raises(ops.WgbError):
        g.dispatch(torch.zeros(8, device="cuda"), m, torch.zeros(255, device="cuda"))
    with pytest.raises(ops.WgbError):
        ops.GpuQuantMatrix(ops.Q4_K, raw, 8, 250)
    with pytest.raises(ops.WgbError):
        ops.GpuQuantMatrix(9, raw, 8, 256)  # Q8_1: unsupported by the reference as well


@pytest.mark.parametrize("qtype", [ops.Q4_K, ops.Q6_K, ops.Q8_0])
def test_gemv_outlier_inputs(qtype):
    """The fast kernels read the input in block fixed point (one exponent per 32 columns, 23 bits).  Inputs that
    stress it: twelve decades inside one 32-column group, groups of zeros, one huge element, denormal-sized
    values -- against the f64 oracle, same tolerance as everywhere."""
    nrows, ncols = 512, 4096
    raw, _ = make(qtype, nrows, ncols, 23)
    rng = np.random.default_rng(5)
    cases = {}
    x = rng.standard_normal(ncols).astype(np.float32)
    x[:32] *= np.float32(10.0) ** rng.uniform(-6, 6, 32).astype(np.float32)      # 12 decades in the first group
    x[32:64] = 0.0                                                                # an all-zero group
    x[64:96] = np.where(np.arange(32) == 7, np.float32(1e4), np.float32(1e-8))    # one outlier among tiny values
    cases["decades"] = x
    x = np.zeros(ncols, np.float32)
    x[1000] = 3.0e30
    x[1001] = -2.5
    cases["one huge element"] = x
    cases["tiny"] = (rng.standard_normal(ncols) * 1e-30).astype(np.float32)
    cases["zeros"] = np.zeros(ncols, np.float32)
    m = ops.GpuQuantMatrix(qtype, raw, nrows, ncols)
    g = ops.GemvQuant.from_device()
    for name, xv in cases.items():
        out = torch.full((nrows,), float("nan"), device="cuda")
        g.dispatch(out, m, torch.from_numpy(xv).cuda())
        o = out.cpu().numpy()
        assert np.isfinite(o).all(), name
        _, o64 = oracle.gemv_quant(qtype, raw, nrows, ncols, xv, want_f64=True)
        atol = ATOL * float(np.sqrt(np.mean(o64 ** 2))) if name != "zeros" else 0.0
        assert_close(o, o64, RTOL, atol, f"qtype {qtype}, {name}")
