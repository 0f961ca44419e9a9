"""wgb_attention_static -- attention on scratch that is part of the library image -- against wgb_attention.

Collected last on purpose (file name): the entry point must give the same result whether it runs alone
in a fresh process or after every other test has used the device.  Each case makes two calls in a row
on the same stream with different inputs, since the second call reuses the scratch and the tickets the
first one left behind."""
import ctypes as C

import numpy as np
import pytest
import torch

from wgml_b200 import _lib
from wgml_b200._lib import AttnParams

pytestmark = pytest.mark.gpu

MAX_FLOATS = 2 * 1024 * 1024
MAX_HEADS = 256


def _case(seed, seq_len, n_heads, kv_mul, head, pos):
    g = torch.Generator(device="cuda").manual_seed(seed)
    kv_dim = n_heads // kv_mul * head
    q = torch.randn(n_heads * head, device="cuda", generator=g)
    k = torch.randn(seq_len, kv_dim, device="cuda", generator=g)
    v = torch.randn(seq_len, kv_dim, device="cuda", generator=g)
    return AttnParams(seq_len, kv_dim, kv_mul, n_heads, head, pos), q, k, v


def _run(fn_static, p, q, k, v):
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    out = torch.full((p.n_heads * p.head_size,), float("nan"), device="cuda")
    if fn_static:
        rc = lib.wgb_attention_static(C.byref(p), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), st)
    else:
        rc = lib.wgb_attention(C.byref(p), q.data_ptr(), k.data_ptr(), v.data_ptr(), None, out.data_ptr(), st)
    _lib.check(rc)
    return out


@pytest.mark.parametrize("shape", [
    dict(seq_len=768, n_heads=32, kv_mul=1, head=128, pos=(540, 17)),      # 7B layout, two different depths
    dict(seq_len=4224, n_heads=64, kv_mul=8, head=128, pos=(4100, 4101)),  # 70B layout, grouped-query
    dict(seq_len=256, n_heads=6, kv_mul=1, head=48, pos=(0, 255)),         # tiny model: first and last position
    # more chunks than one wave of blocks: the streaming kernel (then a short context on the same scratch)
    dict(seq_len=8192, n_heads=32, kv_mul=1, head=128, pos=(8000, 70)),
    dict(seq_len=8192, n_heads=32, kv_mul=2, head=128, pos=(8100, 8101)),  # two query heads per KV head
])
def test_static_matches_allocating_entry_point_twice_in_a_row(shape):
    pos = shape.pop("pos")
    cases = [_case(11 + i, pos=pp, **shape) for i, pp in enumerate(pos)]
    # two calls back to back on one stream, nothing in between
    got = [_run(True, *c) for c in cases]
    torch.cuda.synchronize()
    exp = [_run(False, *c) for c in cases]
    torch.cuda.synchronize()
    for g, e, pp in zip(got, exp, pos):
        assert torch.isfinite(g).all(), f"pos {pp}: output not written"
        assert torch.equal(g, e), f"pos {pp}: max |diff| {float((g - e).abs().max())}"


def test_static_refuses_shapes_beyond_its_scratch():
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    # 64 heads x 132 floats x ceil(seq_len / 64) chunks exceeds 2 Mi floats beyond 15 872 positions
    p, q, k, v = _case(3, seq_len=16000, n_heads=64, kv_mul=8, head=128, pos=5)
    need = p.n_heads * ((p.seq_len + 63) // 64) * (p.head_size + 4)
    assert need > MAX_FLOATS
    out = torch.zeros(p.n_heads * p.head_size, device="cuda")
    rc = lib.wgb_attention_static(C.byref(p), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), st)
    assert rc == _lib.ERR_INVALID
    msg = lib.wgb_last_error().decode()
    assert "scratch" in msg and str(MAX_FLOATS) in msg
    # too many heads
    p2 = AttnParams(64, 512 * 4, 1, 512, 4, 0)
    q2 = torch.zeros(512 * 4, device="cuda")
    kv2 = torch.zeros(64, 512 * 4, device="cuda")
    rc = lib.wgb_attention_static(C.byref(p2), q2.data_ptr(), kv2.data_ptr(), kv2.data_ptr(), q2.clone().data_ptr(), st)
    assert rc == _lib.ERR_INVALID and str(MAX_HEADS) in lib.wgb_last_error().decode()
    # the allocating entry point still serves the large shape
    e = _run(False, p, q, k, v)
    torch.cuda.synchronize()
    assert torch.isfinite(e).all()
