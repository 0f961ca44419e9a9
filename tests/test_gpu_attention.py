"""Decode attention against BatchedMultiqueryAttention::run_cpu (oracle), incl. grouped-query heads,
which the reference never tests."""
import numpy as np
import pytest
import torch

import oracle
from conftest import ATOL, RTOL, assert_close
from wgml_b200 import ops

pytestmark = pytest.mark.gpu


def run(seq_len, n_heads, hs, kv_mul, pos, want_attn, seed=0):
    rng = np.random.default_rng(seed)
    kv_dim = n_heads // kv_mul * hs
    q = rng.standard_normal(n_heads * hs).astype(np.float32)
    kc = rng.standard_normal((seq_len, kv_dim)).astype(np.float32)
    vc = rng.standard_normal((seq_len, kv_dim)).astype(np.float32)
    p = ops.BatchedMultiqueryAttentionParams(seq_len, kv_dim, kv_mul, n_heads, hs, pos)
    xb = torch.full((n_heads * hs,), float("nan"), device="cuda")
    attn = torch.zeros(n_heads * seq_len, device="cuda") if want_attn else None
    a = ops.BatchedMultiqueryAttention.from_device()
    a.dispatch(p, torch.from_numpy(q).cuda(), torch.from_numpy(kc).cuda(), torch.from_numpy(vc).cuda(), attn, xb)
    exb, eattn = oracle.attention(seq_len, kv_dim, kv_mul, n_heads, hs, pos, q, kc, vc)
    assert_close(xb.cpu().numpy(), exb, RTOL, ATOL, f"xb pos={pos} kv_mul={kv_mul}")
    if want_attn:
        got = attn.cpu().numpy().reshape(n_heads, seq_len)
        assert_close(got[:, : pos + 1], eattn[:, : pos + 1], RTOL, 1e-6, "attention weights")
    return xb


@pytest.mark.parametrize("want_attn", [True, False])
def test_reference_test_sizes(want_attn):  # ops/batched_multiquery_attention.rs:210-413
    for pos in list(range(9)):
        run(1024, 12, 64, 1, pos, want_attn, seed=pos)


@pytest.mark.parametrize("case", [
    (256, 6, 48, 1, 255), (768, 32, 128, 1, 600), (4224, 64, 128, 8, 4100), (1024, 12, 64, 1, 1023),
    (512, 12, 64, 3, 130), (512, 16, 32, 2, 63), (512, 16, 32, 2, 64), (512, 10, 256, 5, 77), (128, 4, 4, 4, 100)])
def test_split_kernel_shapes(case):
    run(*case, want_attn=False, seed=1)


@pytest.mark.parametrize("case", [
    (4224, 32, 128, 1, 4100),    # 7B heads, long context: one query head per block, 15 chunks per block
    (4224, 32, 128, 1, 4095),    # last chunk exactly full
    (4224, 32, 128, 4, 4100),    # four query heads per KV head
    (4224, 32, 128, 2, 2049),    # two, last chunk of two positions
    (4224, 40, 128, 5, 3000),    # five query heads share a block of eight
    (4224, 96, 128, 12, 1500),   # twelve: two groups of eight (tail masked)
    (8256, 64, 64, 8, 8200),     # head size 64: half of the lanes idle
    (8256, 24, 96, 1, 5000),     # head size 96
    (4224, 64, 128, 8, 0),       # only the first chunk holds anything, and only one position
    (4224, 64, 128, 8, 63), (4224, 64, 128, 8, 64), (4224, 64, 128, 8, 130),
])
def test_streaming_kernel_shapes(case):
    """Shapes whose chunks outnumber the resident blocks of the split kernel and take the streaming kernel
    (head sizes up to 128): the position bound passed with a host-side `pos` is the position itself."""
    run(*case, want_attn=False, seed=3)


def test_repeated_calls_reuse_the_ticket_counters():
    a = run(512, 8, 64, 2, 300, False, seed=2)
    b = run(512, 8, 64, 2, 300, False, seed=2)
    assert torch.equal(a, b)


def test_repeated_streaming_calls_reuse_the_ticket_counters():
    a = run(4224, 64, 128, 8, 4100, False, seed=4)
    b = run(4224, 64, 128, 8, 4100, False, seed=4)
    assert torch.equal(a, b)


def test_parameter_checks():
    a = ops.BatchedMultiqueryAttention.from_device()
    z = torch.zeros(64 * 128, device="cuda")
    with pytest.raises(ops.WgbError):
        a.dispatch(ops.BatchedMultiqueryAttentionParams(64, 128, 1, 2, 64, 64), z[:128], z, z, None, z[:128])  # pos == seq_len
    with pytest.raises(ops.WgbError):
        a.dispatch(ops.BatchedMultiqueryAttentionParams(64, 128, 3, 2, 64, 1), z[:128], z, z, None, z[:128])
