"""GemvQuant parity for the tcgen05 (tensor memory) Q4_K path through the C ABI: against the oracle's
double-precision product of the same bit-exact weights (1e-3 relative / 1e-4 absolute in units of the output
RMS, as for the CUDA-core kernel) and against the CUDA-core kernel itself."""
import numpy as np
import pytest
import torch

import oracle
from conftest import ATOL, RTOL, assert_close
from wgml_b200 import _lib, ops, synth

pytestmark = pytest.mark.gpu


def make(nrows, ncols, seed):
    qt, arr = synth.matrix(ops.Q4_K, nrows, ncols, seed, "tc")
    x = np.random.default_rng(seed + 1).standard_normal(ncols).astype(np.float32)
    return np.ascontiguousarray(arr).view(np.uint8), x


@pytest.mark.parametrize("shape", [(128, 256), (256, 512), (384, 768), (1280, 4096), (148 * 128 * 2 + 128, 1024)])
def test_tensor_path_vs_oracle(shape):
    nrows, ncols = shape
    raw, x = make(nrows, ncols, 5)
    t = ops.Q4KTiles(raw, nrows, ncols)
    out = torch.full((nrows,), float("nan"), device="cuda")
    t.gemv(out, torch.from_numpy(x).cuda())
    ops.device_status()
    _, o64 = oracle.gemv_quant(ops.Q4_K, raw, nrows, ncols, x, want_f64=True)
    atol = ATOL * max(1.0, float(np.sqrt(np.mean(o64 ** 2))))
    assert_close(out.cpu().numpy(), o64, RTOL, atol, f"tensor path {nrows}x{ncols} vs f64 oracle")


def test_tensor_path_matches_cuda_core_kernel_on_outlier_inputs():
    """Inputs spanning 12 orders of magnitude inside one 32-column group, zeros and a whole zero group."""
    nrows, ncols = 4096, 4096
    raw, _ = make(nrows, ncols, 9)
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(ncols) * 10.0 ** rng.integers(-6, 7, ncols)).astype(np.float32)
    x[64:96] = 0.0
    x[::7] = 0.0
    xd = torch.from_numpy(x).cuda()
    a = torch.zeros(nrows, device="cuda")
    b = torch.zeros(nrows, device="cuda")
    ops.GemvQuant.from_device().dispatch(a, ops.GpuQuantMatrix(ops.Q4_K, raw, nrows, ncols), xd)
    ops.Q4KTiles(raw, nrows, ncols).gemv(b, xd)
    ops.device_status()
    _, o64 = oracle.gemv_quant(ops.Q4_K, raw, nrows, ncols, x, want_f64=True)
    atol = ATOL * float(np.sqrt(np.mean(o64 ** 2)))
    assert_close(b.cpu().numpy(), o64, RTOL, atol, "tensor path, outlier inputs")
    assert_close(b.cpu().numpy(), a.cpu().numpy().astype(np.float64), RTOL, atol, "tensor path vs CUDA-core kernel")


def test_shapes_outside_the_path_are_refused():
    raw, _ = make(128, 256, 1)
    with pytest.raises(_lib.WgbError):
        ops.Q4KTiles(raw[: 100 * 144], 100, 256)            # rows not a multiple of 128
    big, x = make(128, 8192, 1)
    t = ops.Q4KTiles(big, 128, 8192)
    with pytest.raises(_lib.WgbError):                      # more columns than the single-vector kernel's image holds
        t.gemv(torch.zeros(128, device="cuda"), torch.from_numpy(x).cuda())
