"""ctypes binding of libwgml_b200.so (the C ABI declared in include/wgml_b200.h).

The shared object is built in-tree by ``wgml_b200.build``.  There is no fallback: if it is missing
and cannot be built, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("WGML_B200_LIB") or os.path.join(_HERE, "libwgml_b200.so")

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_PARSE, ERR_NOT_FOUND, ERR_TIMEOUT = range(7)
STATUS_NAMES = ["OK", "ERR_INVALID", "ERR_UNSUPPORTED", "ERR_CUDA", "ERR_PARSE", "ERR_NOT_FOUND", "ERR_TIMEOUT"]


class WgbError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else status}: {message}")
        self.status = status
        self.message = message


class RopeConfig(C.Structure):
    """RoPEConfig, crates/wgml/src/ops/rope.rs:26-35."""
    _fields_ = [("head_size", C.c_uint32), ("kv_dim", C.c_uint32), ("pos", C.c_uint32), ("base_freq", C.c_float)]


class AttnParams(C.Structure):
    """BatchedMultiqueryAttentionParams, crates/wgml/src/ops/batched_multiquery_attention.rs:26-37."""
    _fields_ = [("seq_len", C.c_uint32), ("kv_dim", C.c_uint32), ("kv_mul", C.c_uint32), ("n_heads", C.c_uint32),
                ("head_size", C.c_uint32), ("pos", C.c_uint32)]


class Llama2ConfigC(C.Structure):
    """Llama2Config, crates/wgml/src/models/llama2/cpu.rs:46-67."""
    _fields_ = [("dim", C.c_uint32), ("hidden_dim", C.c_uint32), ("n_layers", C.c_uint32), ("n_q_heads", C.c_uint32),
                ("n_kv_heads", C.c_uint32), ("vocab_size", C.c_uint32), ("seq_len", C.c_uint32),
                ("rope_base_freq", C.c_float), ("rms_norm_eps", C.c_float)]


class Gpt2ParamsC(C.Structure):
    """Gpt2Params, crates/wgml/src/models/gpt2/cpu.rs:18-33."""
    _fields_ = [("n_vocab", C.c_uint32), ("n_seq", C.c_uint32), ("n_embd", C.c_uint32), ("n_head", C.c_uint32),
                ("n_layer", C.c_uint32), ("ff_len", C.c_uint32), ("attn_b", C.c_uint32), ("ftype", C.c_uint32)]


class GgufTensorC(C.Structure):
    _fields_ = [("name", C.c_char_p), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 4), ("type", C.c_uint32),
                ("offset", C.c_uint64), ("n_bytes", C.c_uint64), ("data", C.c_void_p)]


_vp, _sz, _i, _u32, _u64, _i64, _f = C.c_void_p, C.c_size_t, C.c_int, C.c_uint32, C.c_uint64, C.c_int64, C.c_float
_pp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes).  Every symbol include/wgml_b200.h declares appears here.
SIGNATURES = {
    "wgb_last_error": (C.c_char_p, []),
    "wgb_version": (C.c_char_p, []),
    "wgb_block_bytes": (_i, [_i]),
    "wgb_block_len": (_i, [_i]),
    "wgb_malloc": (_i, [_pp, _sz]),
    "wgb_free": (_i, [_vp]),
    "wgb_memcpy_h2d": (_i, [_vp, _vp, _sz, _vp]),
    "wgb_memcpy_d2h": (_i, [_vp, _vp, _sz, _vp]),
    "wgb_memset": (_i, [_vp, _i, _sz, _vp]),
    "wgb_stream_synchronize": (_i, [_vp]),
    "wgb_dequantize": (_i, [_i, _vp, _sz, _vp, _vp]),
    "wgb_quant_matrix_create": (_i, [_i, _vp, _sz, _sz, _vp, _pp]),
    "wgb_quant_matrix_create_from_device": (_i, [_i, _vp, _sz, _sz, _vp, _pp]),
    "wgb_quant_matrix_destroy": (_i, [_vp]),
    "wgb_quant_matrix_shape": (_i, [_vp, C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_i)]),
    "wgb_quant_matrix_dequantize_rows": (_i, [_vp, _sz, _sz, _vp, _vp]),
    "wgb_gemv_quant": (_i, [_vp, _vp, _vp, _vp]),
    "wgb_gemv_quant_raw": (_i, [_i, _vp, _sz, _sz, _vp, _vp, _vp]),
    "wgb_q4k_tiles_create": (_i, [_vp, _sz, _sz, _vp, C.POINTER(_vp)]),
    "wgb_q4k_tiles_destroy": (_i, [_vp]),
    "wgb_gemv_q4k_tiles": (_i, [_vp, _vp, _vp, _vp]),
    "wgb_gemm_q4k_tiles": (_i, [_vp, _vp, _sz, _vp, _vp]),
    "wgb_q6k_tiles_create": (_i, [_vp, _sz, _sz, _vp, C.POINTER(_vp)]),
    "wgb_q6k_tiles_destroy": (_i, [_vp]),
    "wgb_gemm_q6k_tiles": (_i, [_vp, _vp, _sz, _vp, _vp]),
    "wgb_q80_tiles_create": (_i, [_vp, _sz, _sz, _vp, C.POINTER(_vp)]),
    "wgb_q80_tiles_destroy": (_i, [_vp]),
    "wgb_gemm_q80_tiles": (_i, [_vp, _vp, _sz, _vp, _vp]),
    "wgb_device_status": (_i, []),
    "wgb_rms_norm": (_i, [_vp, _vp, _vp, _sz, _f, _vp]),
    "wgb_layernorm": (_i, [_vp, _vp, _sz, _vp]),
    "wgb_rope": (_i, [_i, C.POINTER(RopeConfig), _vp, _sz, _vp, _sz, _vp]),
    "wgb_attention": (_i, [C.POINTER(AttnParams), _vp, _vp, _vp, _vp, _vp, _vp]),
    "wgb_attention_static": (_i, [C.POINTER(AttnParams), _vp, _vp, _vp, _vp, _vp]),
    "wgb_softmax": (_i, [_vp, _sz, _sz, _sz, _vp]),
    "wgb_silu": (_i, [_vp, _vp, _sz, _vp]),
    "wgb_unary": (_i, [_i, _vp, _vp, _sz, C.POINTER(_f), _vp]),
    "wgb_unary_inplace": (_i, [_i, _vp, _sz, C.POINTER(_f), _vp]),
    "wgb_op_assign": (_i, [_i, _vp, _vp, _sz, _vp]),
    "wgb_argmax": (_i, [_vp, _sz, _vp, _vp]),
    "wgb_sample": (_i, [_vp, _sz, _f, _f, _f, _vp, _vp]),
    "wgb_sampler_coin": (_f, [_u64, _u64]),
    "wgb_llama2_set_sampler": (_i, [_vp, _f, _f, _u64]),
    "wgb_llama2_load_stats": (_i, [_vp, C.POINTER(_sz), C.POINTER(C.c_double)]),
    "wgb_llama2_set_prefill": (_i, [_vp, _i]),
    "wgb_gpt2_set_prefill": (_i, [_vp, _i]),
    "wgb_gpt2_prefill_positions": (_i, [_vp, C.POINTER(_sz)]),
    "wgb_llama2_prefill_positions": (_i, [_vp, C.POINTER(_sz)]),
    "wgb_gpt2_set_sampler": (_i, [_vp, _f, _f, _u64]),
    "wgb_gguf_open": (_i, [C.c_char_p, _pp]),
    "wgb_gguf_from_bytes": (_i, [_vp, _sz, _pp]),
    "wgb_gguf_close": (_i, [_vp]),
    "wgb_gguf_version": (_u32, [_vp]),
    "wgb_gguf_tensor_count": (_u64, [_vp]),
    "wgb_gguf_metadata_count": (_u64, [_vp]),
    "wgb_gguf_alignment": (_u32, [_vp]),
    "wgb_gguf_meta_find": (_i64, [_vp, C.c_char_p]),
    "wgb_gguf_meta_key": (C.c_char_p, [_vp, _u64]),
    "wgb_gguf_meta_type": (_i, [_vp, _u64, C.POINTER(_i), C.POINTER(_i), C.POINTER(_u64)]),
    "wgb_gguf_meta_u64": (_i, [_vp, _u64, C.POINTER(_u64)]),
    "wgb_gguf_meta_i64": (_i, [_vp, _u64, C.POINTER(_i64)]),
    "wgb_gguf_meta_f64": (_i, [_vp, _u64, C.POINTER(C.c_double)]),
    "wgb_gguf_meta_str": (_i, [_vp, _u64, C.POINTER(_vp), C.POINTER(_u64)]),
    "wgb_gguf_meta_arr_u64": (_i, [_vp, _u64, _u64, C.POINTER(_u64)]),
    "wgb_gguf_meta_arr_i64": (_i, [_vp, _u64, _u64, C.POINTER(_i64)]),
    "wgb_gguf_meta_arr_f64": (_i, [_vp, _u64, _u64, C.POINTER(C.c_double)]),
    "wgb_gguf_meta_arr_str": (_i, [_vp, _u64, _u64, C.POINTER(_vp), C.POINTER(_u64)]),
    "wgb_gguf_tensor_find": (_i64, [_vp, C.c_char_p]),
    "wgb_gguf_tensor_info": (_i, [_vp, _u64, C.POINTER(GgufTensorC)]),
    "wgb_llama_tokenizer_from_gguf": (_i, [_vp, _pp]),
    "wgb_llama_tokenizer_destroy": (_i, [_vp]),
    "wgb_llama_tokenizer_bos": (_u32, [_vp]),
    "wgb_llama_tokenizer_eos": (_u32, [_vp]),
    "wgb_llama_tokenizer_unk": (_u32, [_vp]),
    "wgb_llama_tokenizer_vocab_size": (_sz, [_vp]),
    "wgb_llama_tokenizer_encode": (_i, [_vp, C.c_char_p, _sz, _i, _i, _vp, _sz, C.POINTER(_sz)]),
    "wgb_llama_tokenizer_decode": (_i, [_vp, _u32, _u32, _vp, _sz, C.POINTER(_sz)]),
    "wgb_gpt2_tokenizer_from_gguf": (_i, [_vp, _pp]),
    "wgb_gpt2_tokenizer_destroy": (_i, [_vp]),
    "wgb_gpt2_tokenizer_bos": (_u32, [_vp]),
    "wgb_gpt2_tokenizer_eos": (_u32, [_vp]),
    "wgb_gpt2_tokenizer_encode": (_i, [_vp, C.c_char_p, _sz, _vp, _sz, C.POINTER(_sz)]),
    "wgb_gpt2_tokenizer_decode": (_i, [_vp, _vp, _sz, _vp, _sz, C.POINTER(_sz)]),
    "wgb_chat_template_llama2": (_i, [C.POINTER(C.c_char_p), C.POINTER(C.c_char_p), _sz, C.c_char_p, C.c_char_p, _vp, _sz, C.POINTER(_sz)]),
    "wgb_llama2_config_from_gguf": (_i, [_vp, _i, C.POINTER(Llama2ConfigC)]),
    "wgb_llama2_create": (_i, [C.POINTER(Llama2ConfigC), _i, _i, _i, _pp]),
    "wgb_llama2_destroy": (_i, [_vp]),
    "wgb_llama2_set_matrix": (_i, [_vp, _i, _i, _i, _vp, _sz, _sz]),
    "wgb_llama2_set_vector": (_i, [_vp, _i, _i, _vp, _sz]),
    "wgb_llama2_load_gguf": (_i, [_vp, _vp]),
    "wgb_llama2_set_comm": (_i, [_vp, _vp]),
    "wgb_llama2_set_fused": (_i, [_vp, _i]),
    "wgb_llama2_forward": (_i, [_vp, _u32, _u32, _vp]),
    "wgb_llama2_logits": (_vp, [_vp]),
    "wgb_llama2_x": (_vp, [_vp]),
    "wgb_llama2_key_cache": (_vp, [_vp, _u32]),
    "wgb_llama2_value_cache": (_vp, [_vp, _u32]),
    "wgb_llama2_decode": (_i, [_vp, _vp, _sz, _sz, _u32, _vp, _vp]),
    "wgb_llama2_kernels_per_token": (_i, [_vp]),
    "wgb_llama2_profile_step": (_i, [_vp, _u32, _u32, _vp, _i, C.POINTER(_i), C.POINTER(_i), C.POINTER(_f), C.POINTER(_i)]),
    "wgb_comm_unique_id": (_i, [_vp]),
    "wgb_comm_create": (_i, [_vp, _i, _i, _pp]),
    "wgb_comm_destroy": (_i, [_vp]),
    "wgb_comm_rank": (_i, [_vp]),
    "wgb_comm_size": (_i, [_vp]),
    "wgb_comm_all_reduce_sum": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "wgb_comm_all_gather": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "wgb_comm_shared_alloc": (_i, [_vp, _sz, _pp]),
    "wgb_llama2_set_exchange": (_i, [_vp, _i]),
    "wgb_llama2_set_vocab_shard": (_i, [_vp, _i]),
    "wgb_llama2_exchange_bytes": (_i, [_vp, C.POINTER(_sz), C.POINTER(_sz)]),
    "wgb_llama2_set_exchange_buffers": (_i, [_vp, C.POINTER(_vp), C.POINTER(_vp)]),
    "wgb_set_wait_limit_ms": (_i, [C.c_uint]),
    "wgb_get_wait_limit_ms": (C.c_uint, []),
    "wgb_gpt2_params_from_gguf": (_i, [_vp, C.POINTER(Gpt2ParamsC)]),
    "wgb_gpt2_create": (_i, [C.POINTER(Gpt2ParamsC), _pp]),
    "wgb_gpt2_destroy": (_i, [_vp]),
    "wgb_gpt2_set_matrix": (_i, [_vp, _i, _i, _i, _vp, _sz, _sz]),
    "wgb_gpt2_set_vector": (_i, [_vp, _i, _i, _vp, _sz]),
    "wgb_gpt2_load_gguf": (_i, [_vp, _vp]),
    "wgb_gpt2_set_fused": (_i, [_vp, _i]),
    "wgb_gpt2_forward": (_i, [_vp, _u32, _u32, _vp]),
    "wgb_gpt2_logits": (_vp, [_vp]),
    "wgb_gpt2_key_cache": (_vp, [_vp, _u32]),
    "wgb_gpt2_value_cache": (_vp, [_vp, _u32]),
    "wgb_gpt2_decode": (_i, [_vp, _vp, _sz, _sz, _u32, _vp, _vp]),
    "wgb_gpt2_kernels_per_token": (_i, [_vp]),
}

_lib = None


def load() -> C.CDLL:
    """Loads (building first if needed) the shared library and types its entry points."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        from . import build as _build
        _build.build()
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != OK:
        raise WgbError(status, load().wgb_last_error().decode("utf-8", "replace"))


def last_error() -> str:
    return load().wgb_last_error().decode("utf-8", "replace")
