"""Llama-2 / GPT-2 decoders over the C ABI: the host-side mirror of wgml's `Llama2`, `Llama2Weights`,
`Llama2State`, `Llama2Config` (crates/wgml/src/models/llama2) and `Gpt2*` (crates/wgml/src/models/gpt2)."""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from ._lib import Gpt2ParamsC, Llama2ConfigC, WgbError, check
from .gguf import Gguf
from .ops import require_device


class LlamaModelType(enum.IntEnum):
    """LlamaModelType (crates/wgml/src/models/llama2/mod.rs:14-32)."""
    Llama = 0
    Qwen2 = 1


@dataclass
class Llama2Config:
    """Llama2Config (crates/wgml/src/models/llama2/cpu.rs:46-67)."""
    dim: int
    hidden_dim: int
    n_layers: int
    n_q_heads: int
    n_kv_heads: int
    vocab_size: int
    seq_len: int
    rope_base_freq: float = 10000.0
    rms_norm_eps: float = 1.0e-6

    @classmethod
    def from_gguf(cls, gguf: Gguf, model_type: LlamaModelType = LlamaModelType.Llama) -> "Llama2Config":
        c = Llama2ConfigC()
        check(_lib.load().wgb_llama2_config_from_gguf(gguf._h, int(model_type), C.byref(c)))
        return cls(c.dim, c.hidden_dim, c.n_layers, c.n_q_heads, c.n_kv_heads, c.vocab_size, c.seq_len,
                   c.rope_base_freq, c.rms_norm_eps)

    def to_c(self) -> Llama2ConfigC:
        return Llama2ConfigC(self.dim, self.hidden_dim, self.n_layers, self.n_q_heads, self.n_kv_heads,
                             self.vocab_size, self.seq_len, self.rope_base_freq, self.rms_norm_eps)

    @property
    def head_size(self) -> int:
        return self.dim // self.n_q_heads

    @property
    def kv_dim(self) -> int:
        return self.dim * self.n_kv_heads // self.n_q_heads


LLAMA_MATS = ["attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down"]
LLAMA_VECS = ["attn_norm.weight", "ffn_norm.weight", "attn_q.bias", "attn_k.bias", "attn_v.bias"]


def _np_bytes(a) -> np.ndarray:
    return np.ascontiguousarray(a).view(np.uint8).reshape(-1)


class Llama2:
    """`Llama2` with its weights and state on the current CUDA device.

    `tensors` maps GGUF tensor names to `(ggml_type, ndarray)` (raw blocks or f32 values), the names
    of Llama2Weights::from_gguf (crates/wgml/src/models/llama2/transformer.rs:161-172, 235-237).
    """

    def __init__(self, config: Llama2Config, model_type: LlamaModelType = LlamaModelType.Llama,
                 tp_rank: int = 0, tp_size: int = 1, device=None):
        require_device(device)
        self.config = config
        self.model_type = LlamaModelType(model_type)
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self._h = C.c_void_p()
        c = config.to_c()
        check(_lib.load().wgb_llama2_create(C.byref(c), int(model_type), tp_rank, tp_size, C.byref(self._h)))

    @classmethod
    def new(cls, device, model_type=LlamaModelType.Llama, config: Llama2Config = None):
        return cls(config, model_type, device=device)

    @classmethod
    def from_gguf(cls, gguf: Gguf, model_type=LlamaModelType.Llama, tp_rank=0, tp_size=1) -> "Llama2":
        m = cls(Llama2Config.from_gguf(gguf, model_type), model_type, tp_rank, tp_size)
        check(_lib.load().wgb_llama2_load_gguf(m._h, gguf._h))
        return m

    def load_tensors(self, tensors: dict) -> None:
        lib = _lib.load()
        c = self.config
        shapes = {"attn_q": (c.dim, c.dim), "attn_k": (c.kv_dim, c.dim), "attn_v": (c.kv_dim, c.dim),
                  "attn_output": (c.dim, c.dim), "ffn_gate": (c.hidden_dim, c.dim), "ffn_up": (c.hidden_dim, c.dim),
                  "ffn_down": (c.dim, c.hidden_dim)}
        for l in range(c.n_layers):
            for i, nm in enumerate(LLAMA_MATS):
                qt, arr = tensors[f"blk.{l}.{nm}.weight"]
                raw = _np_bytes(arr)
                check(lib.wgb_llama2_set_matrix(self._h, l, i, qt, raw.ctypes.data, *shapes[nm]))
            for i, nm in enumerate(LLAMA_VECS):
                key = f"blk.{l}.{nm}"
                if key in tensors:
                    v = np.ascontiguousarray(tensors[key][1], dtype=np.float32)
                    check(lib.wgb_llama2_set_vector(self._h, l, i, v.ctypes.data, v.size))
        for which, key in ((0, "token_embd.weight"), (1, "output.weight")):
            if key in tensors:
                qt, arr = tensors[key]
                raw = _np_bytes(arr)
                check(lib.wgb_llama2_set_matrix(self._h, -1, which, qt, raw.ctypes.data, c.vocab_size, c.dim))
        v = np.ascontiguousarray(tensors["output_norm.weight"][1], dtype=np.float32)
        check(lib.wgb_llama2_set_vector(self._h, -1, 0, v.ctypes.data, v.size))

    def load_stats(self) -> tuple[int, float]:
        """(bytes uploaded, seconds the uploads took) so far."""
        b, t = C.c_size_t(), C.c_double()
        check(_lib.load().wgb_llama2_load_stats(self._h, C.byref(b), C.byref(t)))
        return b.value, t.value

    def set_fused(self, enable: bool) -> None:
        check(_lib.load().wgb_llama2_set_fused(self._h, int(enable)))

    def set_comm(self, comm_ptr: int) -> None:
        check(_lib.load().wgb_llama2_set_comm(self._h, comm_ptr))

    def set_exchange(self, mode: int) -> None:
        """0: NCCL all-reduce after attn_output / ffn_down; 1: partial products stored straight into the peers'
        mailboxes by the kernels (collective call: every rank, same mode)."""
        check(_lib.load().wgb_llama2_set_exchange(self._h, int(mode)))

    def set_vocab_shard(self, enable: bool) -> None:
        """Tensor-parallel models: every rank computes vocab_size / tp_size logits and one all-gather per token
        completes them on every rank (collective call: every rank, same setting; needs the communicator)."""
        check(_lib.load().wgb_llama2_set_vocab_shard(self._h, int(enable)))

    def exchange_bytes(self) -> tuple[int, int]:
        """Sizes (mailbox bytes, flag bytes) of one rank's exchange buffers for the direct exchange."""
        a, b = C.c_size_t(), C.c_size_t()
        check(_lib.load().wgb_llama2_exchange_bytes(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def set_exchange_buffers(self, mail_ptrs, flag_ptrs) -> None:
        """Direct exchange over buffers the host mapped itself: entry p is rank p's mailbox / flag array as seen
        from this process (device pointers as ints), entry [tp_rank] this rank's own."""
        n = self.tp_size
        assert len(mail_ptrs) == n and len(flag_ptrs) == n
        mail = (C.c_void_p * n)(*[C.c_void_p(int(p)) for p in mail_ptrs])
        flags = (C.c_void_p * n)(*[C.c_void_p(int(p)) for p in flag_ptrs])
        check(_lib.load().wgb_llama2_set_exchange_buffers(self._h, mail, flags))

    def dispatch(self, token: int, pos: int) -> None:
        """Llama2::dispatch for one token (enqueued on the current stream; logits stay on the device)."""
        check(_lib.load().wgb_llama2_forward(self._h, token, pos, torch.cuda.current_stream().cuda_stream))

    forward = dispatch

    def logits(self) -> torch.Tensor:
        return _device_view(_lib.load().wgb_llama2_logits(self._h), self.config.vocab_size)

    def x(self) -> torch.Tensor:
        return _device_view(_lib.load().wgb_llama2_x(self._h), self.config.dim)

    def _cache(self, ptr: int) -> torch.Tensor:
        """The library keeps a layer's cache head-major, [n_kv_heads][seq_len][head_size]; this returns it in the
        reference's [seq_len][kv_dim] order (a copy)."""
        c = self.config
        kv = c.kv_dim // self.tp_size
        heads = kv // c.head_size
        t = _device_view(ptr, c.seq_len * kv).view(heads, c.seq_len, c.head_size)
        return t.permute(1, 0, 2).reshape(c.seq_len, kv)

    def key_cache(self, layer: int) -> torch.Tensor:
        return self._cache(_lib.load().wgb_llama2_key_cache(self._h, layer))

    def value_cache(self, layer: int) -> torch.Tensor:
        return self._cache(_lib.load().wgb_llama2_value_cache(self._h, layer))

    def decode(self, prompt, n_gen: int, start_pos: int = 0) -> np.ndarray:
        """The token loop (forced prompt tokens, then greedy).  Host ids in, host ids out."""
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        out = np.zeros(max(prompt.size - 1 + n_gen, 1), dtype=np.uint32)
        check(_lib.load().wgb_llama2_decode(self._h, prompt.ctypes.data, prompt.size, n_gen, start_pos, out.ctypes.data,
                                            torch.cuda.current_stream().cuda_stream))
        return out[:prompt.size - 1 + n_gen]

    def set_prefill(self, enable: bool = True) -> None:
        """Batched prompt prefill: `decode` sends the prompt through passes of eight positions with the Q4_K
        products on the tensor cores (the reference feeds it position by position, chat_llama2.rs:104-116)."""
        check(_lib.load().wgb_llama2_set_prefill(self._h, 1 if enable else 0))

    def prefill_positions(self) -> int:
        n = C.c_size_t()
        check(_lib.load().wgb_llama2_prefill_positions(self._h, C.byref(n)))
        return n.value

    def set_sampler(self, temperature: float, topp: float, seed: int = 0) -> None:
        """Sampler::new(vocab, temperature, topp) for the generated tokens of `decode`; temperature 0 = greedy.
        The coin of the token at position p is ops.sampler_coin(seed, p)."""
        check(_lib.load().wgb_llama2_set_sampler(self._h, temperature, topp, seed))

    def kernels_per_token(self) -> int:
        return _lib.load().wgb_llama2_kernels_per_token(self._h)

    PROFILE_KINDS = ["embed", "qkv_rope", "attention", "attn_output", "gate_up_silu", "ffn_down", "logits", "unfused_layer"]

    def profile_step(self, token: int, pos: int):
        """Times every launch of one token forward: list of (kind name, layer, milliseconds).  The fused schedule
        is replayed as the CUDA graph a decode step runs, each launch writing its end time to device memory
        (time = distance to the predecessor's end); the other schedules get an event after every launch."""
        cap = 32 * self.config.n_layers + 16
        kinds, layers, ms, n = (C.c_int * cap)(), (C.c_int * cap)(), (C.c_float * cap)(), C.c_int()
        check(_lib.load().wgb_llama2_profile_step(self._h, token, pos, torch.cuda.current_stream().cuda_stream, cap,
                                                  kinds, layers, ms, C.byref(n)))
        return [(self.PROFILE_KINDS[kinds[i]], layers[i], ms[i]) for i in range(n.value)]

    def close(self):
        if self._h is not None and self._h.value:
            _lib.load().wgb_llama2_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _device_view(ptr: int, n: int) -> torch.Tensor:
    """A float32 CUDA tensor aliasing library-owned device memory (no copy)."""
    if not ptr:
        raise WgbError(_lib.ERR_INVALID, "null device pointer")

    class _Iface:
        __cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 3}

    return torch.as_tensor(_Iface(), device="cuda")


@dataclass
class Gpt2Params:
    """Gpt2Params (crates/wgml/src/models/gpt2/cpu.rs:18-33); defaults = GPT-2 117M (cpu.rs:50-63)."""
    n_vocab: int = 50257
    n_seq: int = 1024
    n_embd: int = 768
    n_head: int = 12
    n_layer: int = 12
    ff_len: int = 3072
    attn_b: int = 2304
    ftype: int = 1

    @classmethod
    def from_gguf(cls, gguf: Gguf) -> "Gpt2Params":
        p = Gpt2ParamsC()
        check(_lib.load().wgb_gpt2_params_from_gguf(gguf._h, C.byref(p)))
        return cls(p.n_vocab, p.n_seq, p.n_embd, p.n_head, p.n_layer, p.ff_len, p.attn_b, p.ftype)

    def to_c(self) -> Gpt2ParamsC:
        return Gpt2ParamsC(self.n_vocab, self.n_seq, self.n_embd, self.n_head, self.n_layer, self.ff_len, self.attn_b, self.ftype)


GPT2_MATS = ["attn_qkv", "attn_output", "ffn_up", "ffn_down"]
GPT2_VECS = ["attn_norm.weight", "attn_norm.bias", "ffn_norm.weight", "ffn_norm.bias", "attn_qkv.bias",
             "attn_output.bias", "ffn_up.bias", "ffn_down.bias"]


class Gpt2:
    """`Gpt2` with weights and state on the device; tensor names as Gpt2Weights::from_gguf
    (crates/wgml/src/models/gpt2/transformer.rs:115-127, 179-188)."""

    def __init__(self, params: Gpt2Params, device=None):
        require_device(device)
        self.params = params
        self._h = C.c_void_p()
        p = params.to_c()
        check(_lib.load().wgb_gpt2_create(C.byref(p), C.byref(self._h)))

    @classmethod
    def from_gguf(cls, gguf: Gguf) -> "Gpt2":
        m = cls(Gpt2Params.from_gguf(gguf))
        check(_lib.load().wgb_gpt2_load_gguf(m._h, gguf._h))
        return m

    def load_tensors(self, tensors: dict) -> None:
        lib = _lib.load()
        p = self.params
        n, ff = p.n_embd, p.ff_len
        shapes = {"attn_qkv": (3 * n, n), "attn_output": (n, n), "ffn_up": (ff, n), "ffn_down": (n, ff)}
        for l in range(p.n_layer):
            for i, nm in enumerate(GPT2_MATS):
                qt, arr = tensors[f"blk.{l}.{nm}.weight"]
                raw = _np_bytes(arr)
                check(lib.wgb_gpt2_set_matrix(self._h, l, i, qt, raw.ctypes.data, *shapes[nm]))
            for i, nm in enumerate(GPT2_VECS):
                v = np.ascontiguousarray(tensors[f"blk.{l}.{nm}"][1], dtype=np.float32)
                check(lib.wgb_gpt2_set_vector(self._h, l, i, v.ctypes.data, v.size))
        for which, key, rows in ((0, "token_embd.weight", p.n_vocab), (1, "position_embd.weight", p.n_seq)):
            qt, arr = tensors[key]
            raw = _np_bytes(arr)
            check(lib.wgb_gpt2_set_matrix(self._h, -1, which, qt, raw.ctypes.data, rows, n))
        for which, key in ((0, "output_norm.weight"), (1, "output_norm.bias")):
            v = np.ascontiguousarray(tensors[key][1], dtype=np.float32)
            check(lib.wgb_gpt2_set_vector(self._h, -1, which, v.ctypes.data, v.size))

    def set_fused(self, enable: bool) -> None:
        check(_lib.load().wgb_gpt2_set_fused(self._h, int(enable)))

    def dispatch(self, embd: int, pos: int) -> None:
        check(_lib.load().wgb_gpt2_forward(self._h, embd, pos, torch.cuda.current_stream().cuda_stream))

    forward = dispatch

    def logits(self) -> torch.Tensor:
        return _device_view(_lib.load().wgb_gpt2_logits(self._h), self.params.n_vocab)

    def key_cache(self, layer: int) -> torch.Tensor:
        p = self.params
        return _device_view(_lib.load().wgb_gpt2_key_cache(self._h, layer), p.n_seq * p.n_embd).view(p.n_seq, p.n_embd)

    def value_cache(self, layer: int) -> torch.Tensor:
        p = self.params
        return _device_view(_lib.load().wgb_gpt2_value_cache(self._h, layer), p.n_seq * p.n_embd).view(p.n_seq, p.n_embd)

    def decode(self, prompt, n_gen: int, start_pos: int = 0) -> np.ndarray:
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        out = np.zeros(max(prompt.size - 1 + n_gen, 1), dtype=np.uint32)
        check(_lib.load().wgb_gpt2_decode(self._h, prompt.ctypes.data, prompt.size, n_gen, start_pos, out.ctypes.data,
                                          torch.cuda.current_stream().cuda_stream))
        return out[:prompt.size - 1 + n_gen]

    def set_sampler(self, temperature: float, topp: float, seed: int = 0) -> None:
        check(_lib.load().wgb_gpt2_set_sampler(self._h, temperature, topp, seed))

    def set_prefill(self, enable: bool = True) -> None:
        """Batched prompt prefill: `decode` sends the prompt through passes of eight positions with the matrix
        products on the tensor cores (the reference feeds it position by position, chat_gpt2.rs:43-151)."""
        check(_lib.load().wgb_gpt2_set_prefill(self._h, 1 if enable else 0))

    def prefill_positions(self) -> int:
        n = C.c_size_t()
        check(_lib.load().wgb_gpt2_prefill_positions(self._h, C.byref(n)))
        return n.value

    def kernels_per_token(self) -> int:
        return _lib.load().wgb_gpt2_kernels_per_token(self._h)

    def close(self):
        if self._h is not None and self._h.value:
            _lib.load().wgb_gpt2_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
