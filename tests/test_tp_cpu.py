"""Tensor-parallel host logic on CPU: the partition rule and a two-rank (gloo) run of the sharded
layer algebra -- head-sharded attention, FFN sharded over the hidden dimension, partial products
summed by all-reduce with the residual folded in by rank 0, and the vocabulary-sharded head completed by an
all-gather -- against the unsharded layer."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from wgml_b200 import tp

CFG = dict(dim=256, hidden_dim=1024, n_q_heads=8, n_kv_heads=4)
VOCAB = 1000
TENSORS = ["attn_q.weight", "attn_k.weight", "attn_v.weight", "attn_output.weight", "ffn_gate.weight",
           "ffn_up.weight", "ffn_down.weight"]


@pytest.mark.parametrize("size", [1, 2, 4, 8])
def test_partition_tiles_every_tensor(size):
    cfg = dict(dim=8192, hidden_dim=28672, n_q_heads=64, n_kv_heads=8)   # Llama-2-70B
    parts = [tp.partition(**cfg, rank=r, size=size) for r in range(size)]
    head = cfg["dim"] // cfg["n_q_heads"]
    for key, total in (("q_rows", cfg["dim"]), ("kv_rows", cfg["n_kv_heads"] * head), ("hidden", cfg["hidden_dim"])):
        edges = [getattr(p, key) for p in parts]
        assert edges[0][0] == 0 and edges[-1][1] == total
        for a, b in zip(edges, edges[1:]):
            assert a[1] == b[0]
        assert all(hi > lo for lo, hi in edges)
    # grouped-query attention stays local: a rank's query heads are exactly those of its KV heads
    for p in parts:
        assert p.n_q_heads == p.n_kv_heads * (cfg["n_q_heads"] // cfg["n_kv_heads"])
        assert p.q_rows[0] // head // (cfg["n_q_heads"] // cfg["n_kv_heads"]) == p.kv_rows[0] // head
        assert p.hidden[0] % 256 == 0 and p.hidden[1] % 256 == 0


def test_partition_rejects_bad_shapes():
    with pytest.raises(ValueError):
        tp.partition(4096, 11008, 32, 32, 0, 3)          # heads do not divide
    with pytest.raises(ValueError):
        tp.partition(4096, 11000, 32, 32, 0, 2)          # hidden_dim not in 256-column blocks
    with pytest.raises(ValueError):
        tp.partition(4096, 11008, 32, 32, 2, 2)          # rank out of range


def _weights(seed=7):
    rng = np.random.default_rng(seed)
    d, h = CFG["dim"], CFG["hidden_dim"]
    head = d // CFG["n_q_heads"]
    kv = CFG["n_kv_heads"] * head
    shapes = {"attn_q.weight": (d, d), "attn_k.weight": (kv, d), "attn_v.weight": (kv, d), "attn_output.weight": (d, d),
              "ffn_gate.weight": (h, d), "ffn_up.weight": (h, d), "ffn_down.weight": (d, h)}
    w = {k: rng.standard_normal(s) / np.sqrt(s[1]) for k, s in shapes.items()}
    w["attn_norm.weight"] = 1.0 + 0.1 * rng.standard_normal(d)
    w["ffn_norm.weight"] = 1.0 + 0.1 * rng.standard_normal(d)
    w["output_norm.weight"] = 1.0 + 0.1 * rng.standard_normal(d)
    w["output.weight"] = rng.standard_normal((VOCAB, d)) / np.sqrt(d)
    return w


def _rms(x, w, eps=1e-5):
    return x / np.sqrt(np.mean(x * x) + eps) * w


def _layer(x, w, n_q, n_kv, kcache, vcache, reduce_sum, is_root):
    """One decoder layer at the position after the cached ones (no RoPE: it acts per head and is
    unaffected by the sharding).  `reduce_sum` sums a vector over the group."""
    head = w["attn_q.weight"].shape[0] // n_q
    xb = _rms(x, w["attn_norm.weight"])
    q, k, v = w["attn_q.weight"] @ xb, w["attn_k.weight"] @ xb, w["attn_v.weight"] @ xb
    kc, vc = np.vstack([kcache, k[None]]), np.vstack([vcache, v[None]])
    out = np.zeros(n_q * head)
    for hq in range(n_q):
        hk = hq // (n_q // n_kv)
        att = kc[:, hk * head:(hk + 1) * head] @ q[hq * head:(hq + 1) * head] / np.sqrt(head)
        att = np.exp(att - att.max())
        att /= att.sum()
        out[hq * head:(hq + 1) * head] = att @ vc[:, hk * head:(hk + 1) * head]
    part = w["attn_output.weight"] @ out
    x = reduce_sum(part + (x if is_root else 0.0))
    xb = _rms(x, w["ffn_norm.weight"])
    g, u = w["ffn_gate.weight"] @ xb, w["ffn_up.weight"] @ xb
    part = w["ffn_down.weight"] @ (u * (g / (1.0 + np.exp(-g))))
    return reduce_sum(part + (x if is_root else 0.0))


def _inputs():
    rng = np.random.default_rng(11)
    head = CFG["dim"] // CFG["n_q_heads"]
    kv = CFG["n_kv_heads"] * head
    return rng.standard_normal(CFG["dim"]), rng.standard_normal((5, kv)), rng.standard_normal((5, kv))


def _rank_main(rank, size, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=size)
    try:
        p = tp.partition(**CFG, rank=rank, size=size)
        full = _weights()
        w = {k: (tp.slice_tensor(k, v, p) if k in TENSORS else v) for k, v in full.items()}
        x, kc, vc = _inputs()

        def reduce_sum(v):
            t = torch.from_numpy(np.ascontiguousarray(v))
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            return t.numpy()

        y = _layer(x, w, p.n_q_heads, p.n_kv_heads, kc[:, p.kv_rows[0]:p.kv_rows[1]], vc[:, p.kv_rows[0]:p.kv_rows[1]],
                   reduce_sum, rank == 0)
        # every rank must end with the same replicated activations
        gathered = [torch.zeros(CFG["dim"], dtype=torch.float64) for _ in range(size)]
        dist.all_gather(gathered, torch.from_numpy(y))
        # vocabulary-sharded head: a rank's run of the logits, completed by an all-gather
        lo, hi = tp.head_rows(VOCAB, rank, size)
        mine = full["output.weight"][lo:hi] @ _rms(y, full["output_norm.weight"])
        runs = [torch.zeros(hi - lo, dtype=torch.float64) for _ in range(size)]
        dist.all_gather(runs, torch.from_numpy(mine))
        if rank == 0:
            np.save(out, np.stack([g.numpy() for g in gathered]))
            np.save(out + ".logits.npy", np.concatenate([r.numpy() for r in runs]))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_rank_layer_matches_unsharded(tmp_path):
    out = str(tmp_path / "y.npy")
    mp.spawn(_rank_main, args=(2, _free_port(), out), nprocs=2, join=True)
    ys = np.load(out)
    x, kc, vc = _inputs()
    ref = _layer(x, _weights(), CFG["n_q_heads"], CFG["n_kv_heads"], kc, vc, lambda v: v, True)
    assert np.array_equal(ys[0], ys[1])
    np.testing.assert_allclose(ys[0], ref, rtol=1e-12, atol=1e-12)
    w = _weights()
    np.testing.assert_allclose(np.load(out + ".logits.npy"), w["output.weight"] @ _rms(ref, w["output_norm.weight"]),
                               rtol=1e-10, atol=1e-10)


def test_head_rows_tile_the_vocabulary():
    for size in (1, 2, 4, 8):
        runs = [tp.head_rows(32000, r, size) for r in range(size)]
        assert runs[0][0] == 0 and runs[-1][1] == 32000
        assert all(a[1] == b[0] for a, b in zip(runs, runs[1:]))
        assert len({hi - lo for lo, hi in runs}) == 1
    with pytest.raises(ValueError):
        tp.head_rows(50257, 0, 2)
    with pytest.raises(ValueError):
        tp.head_rows(32000, 2, 2)


# ---- failure detection on the host: a rank that leaves between steps, a rank that dies silently ------------

def _watch_main(rank, size, port, out_dir, mode):
    """Three steps together; then rank 1 leaves (mode "leave": says good-bye; mode "vanish": just returns)."""
    import datetime
    import time
    store = dist.TCPStore("127.0.0.1", port, size, rank == 0, timeout=datetime.timedelta(seconds=20))
    watch = tp.PeerWatch(store, rank, size, timeout_s=1.0)
    steps_done, error, waited = 0, "", 0.0
    try:
        for step in range(6):
            if rank == 1 and step == 3:
                if mode == "leave":
                    watch.leave()
                break
            t0 = time.monotonic()
            try:
                watch.check()
            finally:
                waited = time.monotonic() - t0
            steps_done += 1          # the launch would go here
    except tp.PeerLost as e:
        error = str(e)
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(f"{steps_done}|{error}|{waited:.3f}")
    if rank == 0:
        time.sleep(0.3)   # the store lives in rank 0: keep it up until rank 1 has written its good-bye


@pytest.mark.parametrize("mode", ["leave", "vanish"])
def test_rank_that_leaves_between_steps_is_an_error_not_a_wait(tmp_path, mode):
    mp.spawn(_watch_main, args=(2, _free_port(), str(tmp_path), mode), nprocs=2, join=True)
    r0 = open(tmp_path / "rank0.txt").read().split("|")
    r1 = open(tmp_path / "rank1.txt").read().split("|")
    assert r1[0] == "3" and r1[1] == ""                     # rank 1 did its three steps and left quietly
    assert r0[0] == "3"                                      # rank 0 launched nothing after the peer was gone
    assert ("left the group" if mode == "leave" else "did not reach step 3") in r0[1]
    assert float(r0[2]) < (0.6 if mode == "leave" else 2.5)  # told at once / after the 1 s limit, never a hang
