"""Bit-exact dequantisation on the GPU, through the C ABI, against the golden vectors and the oracle."""
import numpy as np
import pytest
import torch

import oracle
from conftest import assert_bit_exact
from wgml_b200 import ops, synth

pytestmark = pytest.mark.gpu
QTYPES = [ops.Q4_0, ops.Q4_1, ops.Q5_0, ops.Q5_1, ops.Q8_0, ops.Q4_K, ops.Q5_K, ops.Q6_K, ops.Q8_K]


@pytest.mark.parametrize("qtype", QTYPES)
@pytest.mark.parametrize("kind", ["pattern", "random"])
def test_dequantize_golden(golden, qtype, kind):
    raw = torch.from_numpy(golden[f"{kind}_in_{qtype}"].copy()).cuda()
    got = ops.dequantize(qtype, raw).cpu().numpy()
    assert_bit_exact(got, golden[f"{kind}_out_{qtype}"], f"{kind} {qtype}")


def test_dequantize_f16_every_bit_pattern(golden):
    raw = torch.arange(65536, dtype=torch.int32).to(torch.int16).cuda()
    got = ops.dequantize(ops.F16, raw.view(torch.uint8)).cpu().numpy()
    exp = np.array([oracle.decode_f16(i) for i in range(65536)], dtype=np.float32)
    assert_bit_exact(got, exp, "f16 (NaNs canonical)")


@pytest.mark.parametrize("qtype", QTYPES + [ops.F32])
def test_dequantize_large_random_vs_oracle(qtype):
    rng = np.random.default_rng(qtype)
    nblocks = 4099 if qtype != ops.F32 else 100003  # odd counts: tail handling
    raw = synth.quant_blocks(qtype, nblocks, rng) if qtype != ops.F32 else rng.standard_normal(nblocks).astype(np.float32).view(np.uint8)
    got = ops.dequantize(qtype, torch.from_numpy(raw).cuda()).cpu().numpy()
    assert_bit_exact(got, oracle.dequantize(qtype, raw), f"qtype {qtype}")


def test_dequantize_empty():
    out = ops.dequantize(ops.Q4_K, torch.zeros(0, dtype=torch.uint8, device="cuda"))
    assert out.numel() == 0


@pytest.mark.parametrize("qtype", [ops.Q8_0, ops.Q6_K, ops.Q4_K, ops.Q5_K, ops.F32])
def test_quant_matrix_rows_are_bit_exact_after_repack(qtype):
    """Q8_0 / Q6_K are split into aligned planes at upload; the weights must not change."""
    rng = np.random.default_rng(100 + qtype)
    nrows, ncols = 37, 768
    bl = ops.BLOCK_LEN[qtype]
    raw = synth.quant_blocks(qtype, nrows * ncols // bl, rng) if qtype != ops.F32 else \
        rng.standard_normal(nrows * ncols).astype(np.float32).view(np.uint8)
    exp = oracle.dequantize(qtype, raw).reshape(nrows, ncols)
    for src in (raw, torch.from_numpy(raw).cuda()):  # host upload and device-resident blocks
        m = ops.GpuQuantMatrix(qtype, src, nrows, ncols)
        assert m.shape() == (nrows, ncols)
        assert_bit_exact(m.dequantize_rows(0, nrows).cpu().numpy(), exp, "all rows")
        assert_bit_exact(m.dequantize_rows(5, 3).cpu().numpy(), exp[5:8], "row slice")
    with pytest.raises(ops.WgbError):
        m.dequantize_rows(36, 2)
    with pytest.raises(ops.WgbError):
        ops.GpuQuantMatrix(qtype, raw[:-1], nrows, ncols)
