"""Host-side mirror of wgml's operator structs over the C ABI.

Each class carries the name and call shape of the Rust struct it stands for (``from_device`` builds
it, ``dispatch`` enqueues the kernel on the current CUDA stream and returns at once, shape
mismatches raise where the Rust code asserts).  Buffers are ``torch`` CUDA tensors of dtype
float32: torch is only the owner of device memory and streams here, all arithmetic happens in
libwgml_b200.so.  Views are contiguous slices (``cache[pos]``, ``vec[a:b]``).
"""
from __future__ import annotations

import ctypes as C
import enum

import numpy as np
import torch

from . import _lib
from ._lib import AttnParams as BatchedMultiqueryAttentionParams  # noqa: F401  (re-export)
from ._lib import RopeConfig as RoPEConfig  # noqa: F401
from ._lib import WgbError, check

# ggml tensor type ids (crates/wgml/src/gguf.rs:73-105)
F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q4_K, Q5_K, Q6_K, Q8_K = 0, 1, 2, 3, 6, 7, 8, 12, 13, 14, 15
BLOCK_BYTES = {F32: 4, F16: 2, Q4_0: 18, Q4_1: 20, Q5_0: 22, Q5_1: 24, Q8_0: 34, Q4_K: 144, Q5_K: 176, Q6_K: 210, Q8_K: 292}
BLOCK_LEN = {F32: 1, F16: 1, Q4_0: 32, Q4_1: 32, Q5_0: 32, Q5_1: 32, Q8_0: 32, Q4_K: 256, Q5_K: 256, Q6_K: 256, Q8_K: 256}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _f32(t: torch.Tensor, name: str) -> int:
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
        raise TypeError(f"{name}: expected a contiguous float32 CUDA tensor")
    return t.data_ptr()


def require_device(device=None) -> torch.device:
    """The counterpart of receiving a `&wgpu::Device`: fails loudly without a CUDA device."""
    if not torch.cuda.is_available():
        raise WgbError(_lib.ERR_CUDA, "no CUDA device: wgml_b200 has no CPU path")
    _lib.load()
    return torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)


def dequantize(qtype: int, blocks: torch.Tensor) -> torch.Tensor:
    """Block*::dequantize over a uint8 CUDA tensor of raw GGUF blocks (bit-exact)."""
    require_device()
    raw = blocks.contiguous().view(torch.uint8).reshape(-1)
    nblocks = raw.numel() // BLOCK_BYTES[qtype]
    if nblocks * BLOCK_BYTES[qtype] != raw.numel():
        raise WgbError(_lib.ERR_INVALID, "byte count is not a whole number of blocks")
    out = torch.empty(nblocks * BLOCK_LEN[qtype], dtype=torch.float32, device=raw.device)
    check(_lib.load().wgb_dequantize(qtype, raw.data_ptr(), nblocks, out.data_ptr(), _stream()))
    return out


class GpuQuantMatrix:
    """GpuQuantMatrix (crates/wgml/src/quantized_matrix.rs:9-75), built like
    GgufTensorData::to_gpu_matrix (crates/wgml/src/gguf.rs:131-184) from raw GGUF blocks."""

    def __init__(self, qtype: int, blocks, nrows: int, ncols: int):
        require_device()
        self._h = C.c_void_p()
        lib = _lib.load()
        if isinstance(blocks, torch.Tensor) and blocks.is_cuda:
            raw = blocks.contiguous().view(torch.uint8).reshape(-1)
            self._check_size(qtype, raw.numel(), nrows, ncols)
            check(lib.wgb_quant_matrix_create_from_device(qtype, raw.data_ptr(), nrows, ncols, _stream(), C.byref(self._h)))
            torch.cuda.current_stream().synchronize()
        else:
            raw = np.ascontiguousarray(blocks).view(np.uint8).reshape(-1)
            self._check_size(qtype, raw.size, nrows, ncols)
            check(lib.wgb_quant_matrix_create(qtype, raw.ctypes.data, nrows, ncols, _stream(), C.byref(self._h)))
            torch.cuda.current_stream().synchronize()
        self.qtype, self.nrows, self.ncols = qtype, nrows, ncols

    @staticmethod
    def _check_size(qtype, nbytes, nrows, ncols):
        if qtype not in BLOCK_LEN:
            raise WgbError(_lib.ERR_UNSUPPORTED, f"unsupported tensor type {qtype}")
        if ncols % BLOCK_LEN[qtype] or nbytes != nrows * (ncols // BLOCK_LEN[qtype]) * BLOCK_BYTES[qtype]:
            raise WgbError(_lib.ERR_INVALID, "block bytes do not match nrows x ncols")

    def shape(self):
        return (self.nrows, self.ncols)

    def dequantize_rows(self, row0: int, n: int) -> torch.Tensor:
        out = torch.empty(n * self.ncols, dtype=torch.float32, device="cuda")
        check(_lib.load().wgb_quant_matrix_dequantize_rows(self._h, row0, n, out.data_ptr(), _stream()))
        return out.view(n, self.ncols)

    def __del__(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            _lib.load().wgb_quant_matrix_destroy(self._h)
            self._h = C.c_void_p()


class GemvQuant:
    """GemvQuant (crates/wgml/src/ops/gemv_quant.rs:103-131, 241-348)."""

    @classmethod
    def from_device(cls, device=None):
        require_device(device)
        return cls()

    def dispatch(self, out: torch.Tensor, m: GpuQuantMatrix, v: torch.Tensor) -> None:
        if v.numel() != m.ncols or out.numel() != m.nrows:
            raise WgbError(_lib.ERR_INVALID, "Gemv: dimension mismatch.")
        check(_lib.load().wgb_gemv_quant(m._h, _f32(v, "v"), _f32(out, "out"), _stream()))

    def dispatch_raw(self, out: torch.Tensor, qtype: int, blocks: torch.Tensor, nrows: int, ncols: int, v: torch.Tensor) -> None:
        """The same product over raw GGUF blocks resident on the device."""
        raw = blocks.view(torch.uint8)
        check(_lib.load().wgb_gemv_quant_raw(qtype, raw.data_ptr(), nrows, ncols, _f32(v, "v"), _f32(out, "out"), _stream()))


class Q4KTiles:
    """A Q4_K matrix in the tile-major layout of the tensor-core kernels (nrows a multiple of 128, ncols a
    multiple of 256; the single-vector kernel takes up to 4096 columns), built from raw GGUF blocks in host memory."""

    def __init__(self, blocks, nrows: int, ncols: int):
        require_device()
        raw = np.ascontiguousarray(blocks).view(np.uint8).reshape(-1)
        GpuQuantMatrix._check_size(Q4_K, raw.size, nrows, ncols)
        self._h = C.c_void_p()
        check(_lib.load().wgb_q4k_tiles_create(raw.ctypes.data, nrows, ncols, _stream(), C.byref(self._h)))
        self.nrows, self.ncols = nrows, ncols

    def gemv(self, out: torch.Tensor, v: torch.Tensor) -> None:
        """GemvQuant::dispatch (crates/wgml/src/ops/gemv_quant.rs:241-348) on the tcgen05 path."""
        if v.numel() != self.ncols or out.numel() != self.nrows:
            raise WgbError(_lib.ERR_INVALID, "Gemv: dimension mismatch.")
        check(_lib.load().wgb_gemv_q4k_tiles(self._h, _f32(v, "v"), _f32(out, "out"), _stream()))

    def gemm(self, out: torch.Tensor, v: torch.Tensor) -> None:
        """The product for 1..8 input vectors at once: v [n][ncols] -> out [n][nrows] (the batched prefill's kernel)."""
        if v.dim() != 2 or out.dim() != 2 or v.shape[1] != self.ncols or out.shape[1] != self.nrows or v.shape[0] != out.shape[0]:
            raise WgbError(_lib.ERR_INVALID, "Gemm: dimension mismatch.")
        check(_lib.load().wgb_gemm_q4k_tiles(self._h, _f32(v, "v"), v.shape[0], _f32(out, "out"), _stream()))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _lib.load().wgb_q4k_tiles_destroy(h)
            except Exception:
                pass


class Q6KTiles:
    """A Q6_K matrix in the tile-major layout of the batched tensor-core product (nrows a multiple of 128, ncols
    of 256), built from raw GGUF blocks in host memory."""

    def __init__(self, blocks, nrows: int, ncols: int):
        require_device()
        raw = np.ascontiguousarray(blocks).view(np.uint8).reshape(-1)
        GpuQuantMatrix._check_size(Q6_K, raw.size, nrows, ncols)
        self._h = C.c_void_p()
        check(_lib.load().wgb_q6k_tiles_create(raw.ctypes.data, nrows, ncols, _stream(), C.byref(self._h)))
        self.nrows, self.ncols = nrows, ncols

    def gemm(self, out: torch.Tensor, v: torch.Tensor) -> None:
        """The product for 1..8 input vectors at once: v [n][ncols] -> out [n][nrows]."""
        if v.dim() != 2 or out.dim() != 2 or v.shape[1] != self.ncols or out.shape[1] != self.nrows or v.shape[0] != out.shape[0]:
            raise WgbError(_lib.ERR_INVALID, "Gemm: dimension mismatch.")
        check(_lib.load().wgb_gemm_q6k_tiles(self._h, _f32(v, "v"), v.shape[0], _f32(out, "out"), _stream()))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _lib.load().wgb_q6k_tiles_destroy(h)
            except Exception:
                pass


class Q80Tiles:
    """A Q8_0 matrix in the tile-major layout of the batched tensor-core product (nrows a multiple of 128, ncols
    of 256), built from raw GGUF blocks in host memory."""

    def __init__(self, blocks, nrows: int, ncols: int):
        require_device()
        raw = np.ascontiguousarray(blocks).view(np.uint8).reshape(-1)
        GpuQuantMatrix._check_size(Q8_0, raw.size, nrows, ncols)
        self._h = C.c_void_p()
        check(_lib.load().wgb_q80_tiles_create(raw.ctypes.data, nrows, ncols, _stream(), C.byref(self._h)))
        self.nrows, self.ncols = nrows, ncols

    def gemm(self, out: torch.Tensor, v: torch.Tensor) -> None:
        """The product for 1..8 input vectors at once: v [n][ncols] -> out [n][nrows]."""
        if v.dim() != 2 or out.dim() != 2 or v.shape[1] != self.ncols or out.shape[1] != self.nrows or v.shape[0] != out.shape[0]:
            raise WgbError(_lib.ERR_INVALID, "Gemm: dimension mismatch.")
        check(_lib.load().wgb_gemm_q80_tiles(self._h, _f32(v, "v"), v.shape[0], _f32(out, "out"), _stream()))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _lib.load().wgb_q80_tiles_destroy(h)
            except Exception:
                pass


def device_status() -> None:
    """Waits for the device; raises if a bounded wait inside a matrix-vector kernel has expired."""
    check(_lib.load().wgb_device_status())


class RmsNormConfig:
    """RmsNormConfig (crates/wgml/src/ops/rms_norm.rs:17-21)."""

    def __init__(self, nudge_factor: float):
        self.nudge_factor = float(nudge_factor)


class RmsNorm:
    """RmsNorm (crates/wgml/src/ops/rms_norm.rs:10-63)."""

    @classmethod
    def from_device(cls, device=None):
        require_device(device)
        return cls()

    def dispatch(self, config: RmsNormConfig, result: torch.Tensor, value: torch.Tensor, weight: torch.Tensor) -> None:
        n = value.numel()
        if weight.numel() != n or result.numel() != n:
            raise WgbError(_lib.ERR_INVALID, "RmsNorm: dimension mismatch.")
        check(_lib.load().wgb_rms_norm(_f32(result, "result"), _f32(value, "value"), _f32(weight, "weight"), n,
                                       config.nudge_factor, _stream()))


class LayerNorm:
    """LayerNorm (crates/wgml/src/ops/layernorm.rs:10-54)."""

    @classmethod
    def from_device(cls, device=None):
        require_device(device)
        return cls()

    def dispatch(self, out_vec: torch.Tensor, in_vec: torch.Tensor) -> None:
        if in_vec.numel() != out_vec.numel():
            raise WgbError(_lib.ERR_INVALID, "LayerNorm: dimension mismatch.")  # layernorm.rs:29-33
        check(_lib.load().wgb_layernorm(_f32(out_vec, "out_vec"), _f32(in_vec, "in_vec"), in_vec.numel(), _stream()))


class RoPEVariant(enum.IntEnum):
    """RoPEVariant (crates/wgml/src/ops/rope.rs:10-16)."""
    Original = 0
    Neox = 1


class RoPE:
    """RoPE (crates/wgml/src/ops/rope.rs:18-116)."""

    @classmethod
    def from_device(cls, device=None):
        require_device(device)
        return cls()

    def dispatch(self, variant: RoPEVariant, shape: RoPEConfig, in_out_q: torch.Tensor, in_out_k: torch.Tensor) -> None:
        check(_lib.load().wgb_rope(int(variant), C.byref(shape), _f32(in_out_q, "in_out_q"), in_out_q.numel(),
                                   _f32(in_out_k, "in_out_k"), in_out_k.numel(), _stream()))


class BatchedMultiqueryAttention:
    """BatchedMultiqueryAttention (crates/wgml/src/ops/batched_multiquery_attention.rs:13-195)."""

    @classmethod
    def from_device(cls, device=None):
        require_device(device)
        return cls()

    def dispatch(self, params: BatchedMultiqueryAttentionParams, q, key_cache, value_cache, attn, xb) -> None:
        """`attn` ([n_heads][seq_len]) may be None: the split kernel then runs and no weights are stored."""
        need = params.seq_len * params.kv_dim
        if key_cache.numel() < need or value_cache.numel() < need or q.numel() != params.n_heads * params.head_size \
                or xb.numel() != q.numel() or (attn is not None and attn.numel() < params.n_heads * params.seq_len):
            raise WgbError(_lib.ERR_INVALID, "attention: dimension mismatch.")
        check(_lib.load().wgb_attention(C.byref(params), _f32(q, "q"), _f32(key_cache, "key_cache"),
                                        _f32(value_cache, "value_cache"), None if attn is None else _f32(attn, "attn"),
                                        _f32(xb, "xb"), _stream()))

    # The reference's four-kernel path has the same contract for xb (its attn layout is private).
    dispatch_multi = dispatch


class SoftMax:
    """SoftMax (crates/wgml/src/ops/softmax.rs:10-50): every column of a column-major matrix."""

    @classmethod
    def from_device(cls, device=None):
        require_device(device)
        return cls()

    def dispatch(self, in_out_mat: torch.Tensor, nrows: int | None = None, ncols: int = 1, col_stride: int | None = None) -> None:
        nrows = in_out_mat.numel() if nrows is None else nrows
        col_stride = nrows if col_stride is None else col_stride
        if in_out_mat.numel() < (ncols - 1) * col_stride + nrows:
            raise WgbError(_lib.ERR_INVALID, "softmax: view outside the buffer")
        check(_lib.load().wgb_softmax(_f32(in_out_mat, "in_out_mat"), nrows, ncols, col_stride, _stream()))


class Silu:
    """Silu (crates/wgml/src/ops/silu.rs:10-47)."""

    @classmethod
    def from_device(cls, device=None):
        require_device(device)
        return cls()

    def dispatch(self, in_out_h1: torch.Tensor, in_h2: torch.Tensor) -> None:
        if in_out_h1.numel() != in_h2.numel():
            raise WgbError(_lib.ERR_INVALID, "Silu: dimension mismatch.")
        check(_lib.load().wgb_silu(_f32(in_out_h1, "in_out_h1"), _f32(in_h2, "in_h2"), in_out_h1.numel(), _stream()))


class UnaryOp(enum.IntEnum):
    """UnaryOp (crates/wgml/src/ops/unary.rs:16-38)."""
    Abs = 0
    Sgn = 1
    Neg = 2
    Step = 3
    Elu = 4
    Gelu = 5
    GeluQuick = 6
    Silu = 7
    Tanh = 8
    Relu = 9
    Sigmoid = 10
    HardSigmoid = 11
    HardSwish = 12
    Sqr = 13
    Sqrt = 14
    Log = 15
    LeakyRelu = 16
    Clamp = 17
    Scale = 18
    AddScalar = 19

    def has_args(self) -> bool:
        return self >= UnaryOp.LeakyRelu


def _args4(args):
    if args is None:
        return None
    a = (C.c_float * 4)(*[float(x) for x in list(args) + [0.0] * (4 - len(args))])
    return a


class Unary:
    """Unary (crates/wgml/src/ops/unary.rs:132-203)."""

    def __init__(self, device, op: UnaryOp):
        require_device(device)
        self.op = UnaryOp(op)

    new = classmethod(lambda cls, device, op: cls(device, op))

    def dispatch(self, dest: torch.Tensor, src: torch.Tensor, args=None) -> None:
        if dest.numel() != src.numel():
            raise WgbError(_lib.ERR_INVALID, "Unary: dimension mismatch.")
        check(_lib.load().wgb_unary(int(self.op), _f32(dest, "dest"), _f32(src, "src"), src.numel(), _args4(args), _stream()))


class UnaryInplace:
    """UnaryInplace (crates/wgml/src/ops/unary.rs:205-257)."""

    def __init__(self, device, op: UnaryOp):
        require_device(device)
        self.op = UnaryOp(op)

    new = classmethod(lambda cls, device, op: cls(device, op))

    def dispatch(self, src: torch.Tensor, args=None) -> None:
        check(_lib.load().wgb_unary_inplace(int(self.op), _f32(src, "src"), src.numel(), _args4(args), _stream()))


class OpAssignVariant(enum.IntEnum):
    """wgebra OpAssignVariant as used by wgml (models/llama2/transformer.rs:293, models/gpt2/transformer.rs:259-261)."""
    Add = 0
    Mul = 1
    Copy = 2


class OpAssign:
    def __init__(self, device, variant: OpAssignVariant):
        require_device(device)
        self.variant = OpAssignVariant(variant)

    new = classmethod(lambda cls, device, variant: cls(device, variant))

    def dispatch(self, lhs: torch.Tensor, rhs: torch.Tensor) -> None:
        if lhs.numel() != rhs.numel():
            raise WgbError(_lib.ERR_INVALID, "OpAssign: dimension mismatch.")
        check(_lib.load().wgb_op_assign(int(self.variant), _f32(lhs, "lhs"), _f32(rhs, "rhs"), lhs.numel(), _stream()))


def sample_argmax(v: torch.Tensor) -> int:
    """Sampler::sample_argmax (crates/wgml/src/models/sampler.rs:54-56) evaluated on the device."""
    idx = torch.zeros(1, dtype=torch.int32, device=v.device)
    check(_lib.load().wgb_argmax(_f32(v, "v"), v.numel(), idx.data_ptr(), _stream()))
    return int(idx.item()) & 0xFFFFFFFF


def sampler_coin(seed: int, draw: int) -> float:
    """The uniform draw in [0, 1) the device-resident token loops use for the token at position `draw`."""
    return float(_lib.load().wgb_sampler_coin(seed, draw))


class Sampler:
    """Sampler (crates/wgml/src/models/sampler.rs:14-52) evaluated on the device: the logits never leave it."""

    def __init__(self, vocab_size: int, temperature: float, topp: float):
        self.vocab_size, self.temperature, self.topp = vocab_size, temperature, topp
        self._idx = None

    def sample(self, logits: torch.Tensor, coin: float) -> int:
        """One draw; `coin` in [0, 1) stands for the reference's `random()`."""
        if self._idx is None or self._idx.device != logits.device:
            self._idx = torch.zeros(1, dtype=torch.int32, device=logits.device)
        check(_lib.load().wgb_sample(_f32(logits, "logits"), logits.numel(), self.temperature, self.topp, coin,
                                     self._idx.data_ptr(), _stream()))
        return int(self._idx.item()) & 0xFFFFFFFF
