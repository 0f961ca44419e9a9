"""Tensor parallelism for the Llama-2 token loop: one process per GPU, weights sharded by heads and by
the FFN dimension, two all-reduces per layer.

The reference runs on a single adapter (crates/wgml-bench/src/main.rs:23-36); this module is what lets
a model larger than one GPU's share of work (Llama-2-70B) be served by a group of GPUs.

``partition`` is the single statement of which slice of every tensor a rank keeps; the C library
applies the same rule when a full tensor is uploaded (``wgb_llama2_set_matrix``), and the CPU tests
check that the slices of all ranks tile every tensor and that the sharded computation reproduces the
unsharded one.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import check

COMM_ID_BYTES = 128


@dataclass(frozen=True)
class Partition:
    """Slices kept by one rank.  Row ranges are (start, stop) over output rows, column ranges over
    input columns; everything not listed (embeddings, norms, output matrix) is replicated."""
    rank: int
    size: int
    q_rows: tuple[int, int]        # attn_q rows and attn_output columns
    kv_rows: tuple[int, int]       # attn_k / attn_v rows
    hidden: tuple[int, int]        # ffn_gate / ffn_up rows and ffn_down columns
    n_q_heads: int
    n_kv_heads: int


def partition(dim: int, hidden_dim: int, n_q_heads: int, n_kv_heads: int, rank: int, size: int) -> Partition:
    """Heads are dealt in contiguous runs of n_kv_heads / size KV heads with their query heads (so
    grouped-query attention stays local); the FFN dimension is dealt in 256-column super-blocks, rank r
    taking blocks [nb * r / size, nb * (r + 1) / size)."""
    if not (size >= 1 and 0 <= rank < size):
        raise ValueError(f"bad rank {rank} of {size}")
    if n_kv_heads % size != 0:
        raise ValueError(f"n_kv_heads {n_kv_heads} is not a multiple of the tensor-parallel size {size}")
    if n_q_heads % n_kv_heads != 0 or dim % n_q_heads != 0:
        raise ValueError("head counts do not divide")
    head = dim // n_q_heads
    kv_local = n_kv_heads // size
    q_local = kv_local * (n_q_heads // n_kv_heads)
    if size == 1:
        hid = (0, hidden_dim)
    else:
        if hidden_dim % 256 != 0:
            raise ValueError("tensor parallelism needs hidden_dim % 256 == 0")
        nb = hidden_dim // 256
        hid = (256 * (nb * rank // size), 256 * (nb * (rank + 1) // size))
    return Partition(rank, size, (rank * q_local * head, (rank + 1) * q_local * head),
                     (rank * kv_local * head, (rank + 1) * kv_local * head), hid, q_local, kv_local)


def head_rows(vocab_size: int, rank: int, size: int) -> tuple[int, int]:
    """Rows of the output matrix (= entries of the logits) that rank `rank` computes under the vocabulary-sharded
    head (``Llama2.set_vocab_shard``): equal contiguous runs, so that an all-gather completes the logits."""
    if not (size >= 1 and 0 <= rank < size):
        raise ValueError(f"bad rank {rank} of {size}")
    if vocab_size % size != 0:
        raise ValueError(f"a vocabulary of {vocab_size} rows does not split evenly over {size} ranks")
    n = vocab_size // size
    return rank * n, (rank + 1) * n


def slice_tensor(name: str, full: np.ndarray, p: Partition) -> np.ndarray:
    """The part of a dense [rows, cols] layer tensor that rank p.rank keeps (by GGUF tensor suffix)."""
    if name.endswith("attn_q.weight"):
        return full[p.q_rows[0]:p.q_rows[1]]
    if name.endswith(("attn_k.weight", "attn_v.weight")):
        return full[p.kv_rows[0]:p.kv_rows[1]]
    if name.endswith("attn_output.weight"):
        return full[:, p.q_rows[0]:p.q_rows[1]]
    if name.endswith(("ffn_gate.weight", "ffn_up.weight")):
        return full[p.hidden[0]:p.hidden[1]]
    if name.endswith("ffn_down.weight"):
        return full[:, p.hidden[0]:p.hidden[1]]
    if name.endswith("attn_q.bias"):
        return full[p.q_rows[0]:p.q_rows[1]]
    if name.endswith(("attn_k.bias", "attn_v.bias")):
        return full[p.kv_rows[0]:p.kv_rows[1]]
    return full


class Comm:
    """The tensor-parallel group of this process (``wgb_comm``)."""

    def __init__(self, unique_id: bytes, rank: int, size: int):
        if len(unique_id) != COMM_ID_BYTES:
            raise ValueError("a communicator id has 128 bytes")
        self._h = C.c_void_p()
        buf = C.create_string_buffer(unique_id, COMM_ID_BYTES)
        check(_lib.load().wgb_comm_create(buf, rank, size, C.byref(self._h)))
        self.rank, self.size = rank, size

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(COMM_ID_BYTES)
        check(_lib.load().wgb_comm_unique_id(buf))
        return buf.raw

    @property
    def handle(self) -> int:
        return self._h.value

    def all_reduce_sum(self, send, recv=None) -> None:
        """In-place (recv None) or out-of-place sum of a float32 CUDA tensor over the group."""
        import torch
        recv = send if recv is None else recv
        assert send.dtype == torch.float32 and recv.dtype == torch.float32 and send.numel() == recv.numel()
        check(_lib.load().wgb_comm_all_reduce_sum(self._h, send.data_ptr(), recv.data_ptr(), send.numel(),
                                                  torch.cuda.current_stream().cuda_stream))

    def close(self) -> None:
        if self._h:
            _lib.load().wgb_comm_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def init_from_torch_distributed() -> Comm:
    """Builds the group over the ranks of an initialised torch.distributed process group: rank 0 makes
    the id and broadcasts it (any backend; the payload is 128 bytes)."""
    import torch
    import torch.distributed as dist
    rank, size = dist.get_rank(), dist.get_world_size()
    box = [Comm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    return Comm(box[0], rank, size)


def set_wait_limit_ms(ms: int) -> None:
    """How long a kernel waits for the other ranks' flags before the decode call fails with a time-out
    (process-wide; default 2000 ms)."""
    check(_lib.load().wgb_set_wait_limit_ms(int(ms)))


class PeerLost(RuntimeError):
    """A rank of the group has left or stopped answering; raised on the host, before anything is launched."""


class PeerWatch:
    """Host-side liveness of a tensor-parallel group, checked between decode calls.

    The kernels of the direct exchange wait for one another on the device, so a rank must never launch a
    step that a peer will not join.  Every rank publishes the number of the step it is about to launch in a
    key-value store shared by the group (any ``torch.distributed`` store: the TCPStore of the rendezvous, a
    FileStore, ...) and, before launching, waits at most `timeout_s` for every peer to have published the same
    step.  A rank that leaves in an orderly way says so (`leave`), and its peers learn of it at their next
    check without waiting.  No device is involved; the device-side wait limit (`set_wait_limit_ms`) stays as
    the second line of defence for a rank that dies in the middle of a step."""

    def __init__(self, store, rank: int, size: int, timeout_s: float = 5.0, prefix: str = "wgb_tp"):
        self.store, self.rank, self.size, self.timeout_s, self.prefix = store, rank, size, timeout_s, prefix
        self.step = 0

    def _key(self, kind: str, rank: int, step: int | None = None) -> str:
        return f"{self.prefix}/{kind}/{rank}" + ("" if step is None else f"/{step}")

    def check(self) -> int:
        """Call before every launch (decode call).  Returns the step number; raises PeerLost."""
        import datetime
        step = self.step
        try:
            self.store.set(self._key("step", self.rank, step), b"1")
            for p in range(self.size):
                if p == self.rank:
                    continue
                if self.store.check([self._key("left", p)]):
                    raise PeerLost(f"rank {p} left the group before step {step}")
            keys = [self._key("step", p, step) for p in range(self.size) if p != self.rank]
            if keys:
                deadline = datetime.timedelta(seconds=self.timeout_s)
                # poll in short slices so that a rank that says good-bye while we wait is noticed at once
                import time
                t_end = time.monotonic() + self.timeout_s
                while True:
                    try:
                        self.store.wait(keys, min(deadline, datetime.timedelta(milliseconds=100)))
                        break
                    except PeerLost:
                        raise
                    except Exception:
                        for p in range(self.size):
                            if p != self.rank and self.store.check([self._key("left", p)]):
                                raise PeerLost(f"rank {p} left the group before step {step}")
                        if time.monotonic() >= t_end:
                            missing = [p for p in range(self.size) if p != self.rank
                                       and not self.store.check([self._key("step", p, step)])]
                            raise PeerLost(f"ranks {missing} did not reach step {step} within {self.timeout_s} s")
        except PeerLost:
            raise
        except Exception as e:   # the store itself is gone (its host rank died)
            raise PeerLost(f"the group's store stopped answering at step {step}: {e}") from e
        self.step += 1
        return step

    def leave(self) -> None:
        """Tells the peers that this rank will launch nothing more (call between steps, nothing in flight)."""
        try:
            self.store.set(self._key("left", self.rank), b"1")
        except Exception:
            pass


def guarded_decode(model, watch: PeerWatch, prompt, n_gen: int, start_pos: int = 0):
    """``model.decode`` preceded by the group's liveness check: raises PeerLost instead of launching a step that
    a peer will not join."""
    watch.check()
    return model.decode(prompt, n_gen, start_pos=start_pos)


def attach(model, comm: Comm, direct: bool = True, vocab_shard: bool = False) -> None:
    """Gives a tensor-parallel ``Llama2`` its group; must precede the first forward.  `direct`: the kernels
    exchange partial products through peer memory themselves instead of calling NCCL's all-reduce.
    `vocab_shard`: every rank computes its run of the logits and an all-gather completes them."""
    model.set_comm(comm.handle)
    model._comm = comm   # keep it alive as long as the model
    model.set_exchange(1 if direct else 0)
    model.set_vocab_shard(vocab_shard)
