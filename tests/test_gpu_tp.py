"""Tensor-parallel Llama-2 on 2 GPUs against the same model on one GPU: identical greedy tokens and
logits within 1e-3 relative / 1e-4 absolute (absolute term scaled by the largest logit), for the direct
exchange of partial products through peer memory and for the NCCL all-reduce, with the replicated and the
vocabulary-sharded output head.  Needs two devices; skipped
otherwise.  The ranks are separate processes over NCCL, as in production."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ATOL, RTOL, assert_close

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp2_matches_single_gpu(tmp_path):
    out = str(tmp_path / "tp.npz")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(HERE, "tp_worker.py"), out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = np.load(out)
    for name in ("gqa_q4k", "tiny_f32"):
        ref_t, ref_l = res[f"{name}/ref_tokens"], res[f"{name}/ref_logits"]
        for mode in ("11", "10", "00"):   # fused + direct exchange, fused + NCCL, dispatch by dispatch + NCCL
            assert np.array_equal(res[f"{name}/{mode}/tp_tokens"], ref_t), f"{name} mode {mode}: tokens differ"
            scale = max(1.0, float(np.abs(ref_l).max()))
            assert_close(res[f"{name}/{mode}/tp_logits"], ref_l, RTOL, ATOL * scale, f"{name} mode {mode} logits")
            ref_x = res[f"{name}/ref_x"]
            assert_close(res[f"{name}/{mode}/tp_x"], ref_x, RTOL, ATOL * max(1.0, float(np.abs(ref_x).max())),
                         f"{name} mode {mode} residual stream")
        for mode in ("11", "00"):   # vocabulary-sharded head: same tokens, same full logits on rank 0
            assert np.array_equal(res[f"{name}/vs{mode}/tp_tokens"], ref_t), f"{name} vocab shard {mode}: tokens differ"
            assert_close(res[f"{name}/vs{mode}/tp_logits"], ref_l, RTOL, ATOL * max(1.0, float(np.abs(ref_l).max())),
                         f"{name} vocab shard {mode} logits")
    # batched prompt passes on the sharded model against the unsharded position-by-position loop
    ref_t, ref_l = res["gqa_q4k/prefill/ref_tokens"], res["gqa_q4k/prefill/ref_logits"]
    for mode in ("1", "0"):
        assert np.array_equal(res[f"gqa_q4k/prefill{mode}/tp_tokens"], ref_t), f"prefill, exchange {mode}: tokens differ"
        assert_close(res[f"gqa_q4k/prefill{mode}/tp_logits"], ref_l, RTOL, ATOL * max(1.0, float(np.abs(ref_l).max())),
                     f"prefill, exchange {mode}: logits after the last step")
