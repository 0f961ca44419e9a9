"""CPU oracle for the wgml token-loop path: numpy-facing bindings of ``wgml_oracle.c``.

TEST INFRASTRUCTURE ONLY.  Importers are limited to ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``; the product package never imports
this module.  The C file cites, function by function, the wgml source it restates.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libwgml_oracle.so")
_lib = None

# ggml tensor type ids (crates/wgml/src/gguf.rs:73-105)
F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q4_K, Q5_K, Q6_K, Q8_K = 0, 1, 2, 3, 6, 7, 8, 12, 13, 14, 15
QTYPE_NAMES = {F32: "F32", F16: "F16", Q4_0: "Q4_0", Q4_1: "Q4_1", Q5_0: "Q5_0", Q5_1: "Q5_1",
               Q8_0: "Q8_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K", Q8_K: "Q8_K"}
BLOCK_BYTES = {F32: 4, F16: 2, Q4_0: 18, Q4_1: 20, Q5_0: 22, Q5_1: 24, Q8_0: 34, Q4_K: 144,
               Q5_K: 176, Q6_K: 210, Q8_K: 292}
BLOCK_LEN = {F32: 1, F16: 1, Q4_0: 32, Q4_1: 32, Q5_0: 32, Q5_1: 32, Q8_0: 32, Q4_K: 256,
             Q5_K: 256, Q6_K: 256, Q8_K: 256}

# UnaryOp numbering = enum order of crates/wgml/src/ops/unary.rs:16-38
UNARY_OPS = ["Abs", "Sgn", "Neg", "Step", "Elu", "Gelu", "GeluQuick", "Silu", "Tanh", "Relu",
             "Sigmoid", "HardSigmoid", "HardSwish", "Sqr", "Sqrt", "Log", "LeakyRelu", "Clamp",
             "Scale", "AddScalar"]


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (see Makefile).  Returns the path of the shared object."""
    src = os.path.join(_HERE, "wgml_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        cmd = ["make", "-C", _HERE, "-s", "-B"]
        if subprocess.run(cmd, capture_output=True).returncode != 0:
            subprocess.run(cmd + ["OPENMP="], check=True)  # no libgomp: single-threaded oracle
    return _SO


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        f32p, u32p, vp = C.POINTER(C.c_float), C.POINTER(C.c_uint32), C.c_void_p
        sz = C.c_size_t
        L.wgo_decode_f16.restype = C.c_float
        L.wgo_decode_f16.argtypes = [C.c_uint16]
        L.wgo_dequantize.argtypes = [C.c_int, vp, sz, vp]
        L.wgo_gemv_quant.argtypes = [C.c_int, vp, sz, sz, vp, vp, vp]
        L.wgo_rms_norm.argtypes = [vp, vp, vp, sz, C.c_float]
        L.wgo_layernorm.argtypes = [vp, vp, sz]
        L.wgo_rope.argtypes = [C.c_int, vp, sz, vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float]
        L.wgo_softmax.argtypes = [vp, sz]
        L.wgo_silu.argtypes = [vp, vp, sz]
        L.wgo_unary_vec.argtypes = [C.c_int, vp, sz, vp]
        L.wgo_attention.argtypes = [vp, vp, vp, vp, vp, vp]
        L.wgo_argmax.restype = sz
        L.wgo_argmax.argtypes = [vp, sz]
        L.wgo_llama2_new.restype = vp
        L.wgo_llama2_new.argtypes = [C.c_uint32] * 7 + [C.c_float, C.c_float, C.c_int]
        L.wgo_llama2_free.argtypes = [vp]
        L.wgo_llama2_set_matrix.argtypes = [vp, C.c_int, C.c_int, C.c_int, vp, sz, sz]
        L.wgo_llama2_set_vector.argtypes = [vp, C.c_int, C.c_int, vp]
        for name in ("logits", "key_cache", "value_cache", "x"):
            fn = getattr(L, "wgo_llama2_" + name)
            fn.restype, fn.argtypes = f32p, [vp]
        L.wgo_llama2_forward.argtypes = [vp, C.c_uint32, C.c_uint32]
        L.wgo_llama2_layer_forward.argtypes = [vp, C.c_uint32, C.c_uint32]
        L.wgo_llama2_head_forward.argtypes = [vp]
        L.wgo_llama2_decode.argtypes = [vp, vp, sz, sz, C.c_uint32, vp, vp]
        L.wgo_gpt2_new.restype = vp
        L.wgo_gpt2_new.argtypes = [C.c_uint32] * 6
        L.wgo_gpt2_free.argtypes = [vp]
        L.wgo_gpt2_set_matrix.argtypes = [vp, C.c_int, C.c_int, C.c_int, vp, sz, sz]
        L.wgo_gpt2_set_vector.argtypes = [vp, C.c_int, C.c_int, vp]
        for name in ("logits", "key_cache", "value_cache"):
            fn = getattr(L, "wgo_gpt2_" + name)
            fn.restype, fn.argtypes = f32p, [vp]
        L.wgo_gpt2_forward.argtypes = [vp, C.c_uint32, C.c_uint32]
        L.wgo_gpt2_decode.argtypes = [vp, vp, sz, sz, C.c_uint32, vp]
        L.wgo_num_threads.restype = C.c_int
        L.wgo_set_num_threads.argtypes = [C.c_int]
        L.wgo_set_dot_f64.argtypes = [C.c_int]
        L.wgo_sampler_coin.restype = C.c_float
        L.wgo_sampler_coin.argtypes = [C.c_uint64, C.c_uint64]
        L.wgo_sample.restype = C.c_size_t
        L.wgo_sample.argtypes = [vp, sz, C.c_float, C.c_float, C.c_float, vp]
        _lib = L
    return _lib


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def set_num_threads(n: int) -> None:
    lib().wgo_set_num_threads(int(n))


def set_dot_f64(on: bool) -> None:
    """Accumulate every matrix-vector product of the transformers in double (rounded to f32 once): the gap to
    the default f32 accumulation measures how far summation rounding alone moves a model's logits."""
    lib().wgo_set_dot_f64(int(bool(on)))


def num_threads() -> int:
    return int(lib().wgo_num_threads())


def decode_f16(bits: int) -> np.float32:
    return np.float32(lib().wgo_decode_f16(int(bits) & 0xFFFF))


def dequantize(qtype: int, blocks: np.ndarray) -> np.ndarray:
    """Raw GGUF block bytes (uint8) -> f32 values, block after block."""
    raw = np.ascontiguousarray(blocks).view(np.uint8).ravel()
    nblocks = raw.size // BLOCK_BYTES[qtype]
    assert nblocks * BLOCK_BYTES[qtype] == raw.size
    out = np.empty(nblocks * BLOCK_LEN[qtype], dtype=np.float32)
    rc = lib().wgo_dequantize(qtype, _p(raw), nblocks, _p(out))
    assert rc == 0
    return out


def gemv_quant(qtype: int, w: np.ndarray, nrows: int, ncols: int, x: np.ndarray, want_f64=False):
    raw = np.ascontiguousarray(w).view(np.uint8).ravel()
    x = _f32(x)
    assert x.size == ncols
    assert raw.size == nrows * (ncols // BLOCK_LEN[qtype]) * BLOCK_BYTES[qtype]
    out = np.empty(nrows, dtype=np.float32)
    out64 = np.empty(nrows, dtype=np.float64) if want_f64 else None
    rc = lib().wgo_gemv_quant(qtype, _p(raw), nrows, ncols, _p(x), _p(out),
                              _p(out64) if want_f64 else None)
    assert rc == 0
    return (out, out64) if want_f64 else out


def rms_norm(a, w, eps=1.0e-5) -> np.ndarray:
    a, w = _f32(a), _f32(w)
    out = np.empty_like(a)
    lib().wgo_rms_norm(_p(out), _p(a), _p(w), a.size, eps)
    return out


def layernorm(v) -> np.ndarray:
    v = _f32(v)
    out = np.empty_like(v)
    lib().wgo_layernorm(_p(out), _p(v), v.size)
    return out


def rope(variant: int, q, k, head_size: int, kv_dim: int, pos: int, base=10000.0):
    """Returns rotated copies (q, k)."""
    q, k = _f32(q).copy(), _f32(k).copy()
    lib().wgo_rope(variant, _p(q), q.size, _p(k), head_size, kv_dim, pos, base)
    return q, k


def softmax(v) -> np.ndarray:
    v = _f32(v).copy()
    lib().wgo_softmax(_p(v), v.size)
    return v


def silu(h1, h2) -> np.ndarray:
    h1, h2 = _f32(h1).copy(), _f32(h2)
    lib().wgo_silu(_p(h1), _p(h2), h1.size)
    return h1


def unary(op: int, v, args=(0.0, 0.0, 0.0, 0.0)) -> np.ndarray:
    v = _f32(v).copy()
    a = np.asarray(args, dtype=np.float32)
    lib().wgo_unary_vec(op, _p(v), v.size, _p(a))
    return v


def attention(seq_len, kv_dim, kv_mul, n_heads, head_size, pos, q, key_cache, value_cache):
    """Caches: float32 [seq_len][kv_dim].  Returns (xb, attn[n_heads][seq_len])."""
    params = np.array([seq_len, kv_dim, kv_mul, n_heads, head_size, pos], dtype=np.uint32)
    q, kc, vc = _f32(q), _f32(key_cache), _f32(value_cache)
    attn = np.zeros((n_heads, seq_len), dtype=np.float32)
    xb = np.zeros(n_heads * head_size, dtype=np.float32)
    lib().wgo_attention(_p(params), _p(q), _p(kc), _p(vc), _p(attn), _p(xb))
    return xb, attn


def sampler_coin(seed: int, draw: int) -> float:
    return float(lib().wgo_sampler_coin(seed, draw))


def sample(logits, temperature: float, topp: float, coin: float):
    """Sampler::sample (crates/wgml/src/models/sampler.rs:32-52).  Returns (token, slack): slack is how far the
    deciding comparison was from its threshold, relative to the probability mass walked."""
    a = _f32(logits).copy()
    sl = np.zeros(1, np.float32)
    tok = lib().wgo_sample(_p(a), a.size, float(temperature), float(topp), float(coin), _p(sl))
    return int(tok), float(sl[0])


def argmax(v) -> int:
    v = _f32(v)
    return int(lib().wgo_argmax(_p(v), v.size))


LLAMA_MATS = ["attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down"]
LLAMA_VECS = ["attn_norm", "ffn_norm", "attn_q.bias", "attn_k.bias", "attn_v.bias"]


class Llama2Oracle:
    """CPU Llama-2 transformer over a dict of GGUF-named tensors.

    ``tensors[name] = (qtype, ndarray)``; matrices are raw block bytes (or f32 values), vectors
    f32.  Names follow crates/wgml/src/models/llama2/transformer.rs:161-172,235-237.
    """

    def __init__(self, cfg: dict, tensors: dict, rope_variant: int = 0):
        L = lib()
        self.cfg = cfg
        self._keep = []
        self.h = L.wgo_llama2_new(cfg["dim"], cfg["hidden_dim"], cfg["n_layers"], cfg["n_q_heads"],
                                  cfg["n_kv_heads"], cfg["vocab_size"], cfg["seq_len"],
                                  cfg.get("rope_base_freq", 10000.0), cfg.get("rms_norm_eps", 1e-5),
                                  rope_variant)
        dim, hid = cfg["dim"], cfg["hidden_dim"]
        kv_dim = dim * cfg["n_kv_heads"] // cfg["n_q_heads"]
        shapes = {"attn_q": (dim, dim), "attn_k": (kv_dim, dim), "attn_v": (kv_dim, dim),
                  "attn_output": (dim, dim), "ffn_gate": (hid, dim), "ffn_up": (hid, dim),
                  "ffn_down": (dim, hid)}
        for l in range(cfg["n_layers"]):
            for i, nm in enumerate(LLAMA_MATS):
                qt, arr = tensors[f"blk.{l}.{nm}.weight"]
                self._set_mat(l, i, qt, arr, *shapes[nm])
            for i, nm in enumerate(LLAMA_VECS):
                key = f"blk.{l}.{nm}" if nm.endswith(".bias") else f"blk.{l}.{nm}.weight"
                if key in tensors:
                    self._set_vec(l, i, tensors[key][1])
        qt, arr = tensors["token_embd.weight"]
        self._set_mat(-1, 0, qt, arr, cfg["vocab_size"], dim)
        qt, arr = tensors.get("output.weight", tensors["token_embd.weight"])
        self._set_mat(-1, 1, qt, arr, cfg["vocab_size"], dim)
        self._set_vec(-1, 0, tensors["output_norm.weight"][1])

    def _set_mat(self, layer, which, qt, arr, nrows, ncols):
        a = np.ascontiguousarray(arr)
        self._keep.append(a)
        lib().wgo_llama2_set_matrix(self.h, layer, which, qt, _p(a), nrows, ncols)

    def _set_vec(self, layer, which, arr):
        a = _f32(arr)
        self._keep.append(a)
        lib().wgo_llama2_set_vector(self.h, layer, which, _p(a))

    def forward(self, token: int, pos: int) -> np.ndarray:
        lib().wgo_llama2_forward(self.h, token, pos)
        return self.logits()

    def layer_forward(self, layer: int, pos: int) -> None:
        """One layer on the running activation (timing samples of large models)."""
        lib().wgo_llama2_layer_forward(self.h, layer, pos)

    def head_forward(self) -> None:
        lib().wgo_llama2_head_forward(self.h)

    def logits(self) -> np.ndarray:
        return np.ctypeslib.as_array(lib().wgo_llama2_logits(self.h), (self.cfg["vocab_size"],)).copy()

    def x(self) -> np.ndarray:
        return np.ctypeslib.as_array(lib().wgo_llama2_x(self.h), (self.cfg["dim"],)).copy()

    def caches(self):
        c = self.cfg
        kv_dim = c["dim"] * c["n_kv_heads"] // c["n_q_heads"]
        shp = (c["n_layers"], c["seq_len"], kv_dim)
        return (np.ctypeslib.as_array(lib().wgo_llama2_key_cache(self.h), shp),
                np.ctypeslib.as_array(lib().wgo_llama2_value_cache(self.h), shp))

    def decode(self, prompt, n_gen: int, start_pos: int = 0):
        """Returns (tokens, top2_margins); tokens[i] is the token fed at position start_pos+i+1."""
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        total = prompt.size - 1 + n_gen
        out = np.zeros(total, dtype=np.uint32)
        margin = np.zeros(total, dtype=np.float32)
        lib().wgo_llama2_decode(self.h, _p(prompt), prompt.size, n_gen, start_pos, _p(out), _p(margin))
        return out, margin

    def __del__(self):
        if getattr(self, "h", None):
            lib().wgo_llama2_free(self.h)
            self.h = None


GPT2_MATS = ["attn_qkv", "attn_output", "ffn_up", "ffn_down"]
GPT2_VECS = ["attn_norm.weight", "attn_norm.bias", "ffn_norm.weight", "ffn_norm.bias",
             "attn_qkv.bias", "attn_output.bias", "ffn_up.bias", "ffn_down.bias"]


class Gpt2Oracle:
    """CPU GPT-2 transformer; tensor names as crates/wgml/src/models/gpt2/cpu.rs:118-130,180-189."""

    def __init__(self, cfg: dict, tensors: dict):
        L = lib()
        self.cfg = cfg
        self._keep = []
        n, ff = cfg["n_embd"], cfg["ff_len"]
        self.h = L.wgo_gpt2_new(cfg["n_vocab"], cfg["n_seq"], n, cfg["n_head"], cfg["n_layer"], ff)
        shapes = {"attn_qkv": (3 * n, n), "attn_output": (n, n), "ffn_up": (ff, n), "ffn_down": (n, ff)}
        for l in range(cfg["n_layer"]):
            for i, nm in enumerate(GPT2_MATS):
                qt, arr = tensors[f"blk.{l}.{nm}.weight"]
                self._set_mat(l, i, qt, arr, *shapes[nm])
            for i, nm in enumerate(GPT2_VECS):
                self._set_vec(l, i, tensors[f"blk.{l}.{nm}"][1])
        qt, arr = tensors["token_embd.weight"]
        self._set_mat(-1, 0, qt, arr, cfg["n_vocab"], n)
        qt, arr = tensors["position_embd.weight"]
        self._set_mat(-1, 1, qt, arr, cfg["n_seq"], n)
        self._set_vec(-1, 0, tensors["output_norm.weight"][1])
        self._set_vec(-1, 1, tensors["output_norm.bias"][1])

    def _set_mat(self, layer, which, qt, arr, nrows, ncols):
        a = np.ascontiguousarray(arr)
        self._keep.append(a)
        lib().wgo_gpt2_set_matrix(self.h, layer, which, qt, _p(a), nrows, ncols)

    def _set_vec(self, layer, which, arr):
        a = _f32(arr)
        self._keep.append(a)
        lib().wgo_gpt2_set_vector(self.h, layer, which, _p(a))

    def forward(self, token: int, pos: int) -> np.ndarray:
        lib().wgo_gpt2_forward(self.h, token, pos)
        return np.ctypeslib.as_array(lib().wgo_gpt2_logits(self.h), (self.cfg["n_vocab"],)).copy()

    def caches(self):
        c = self.cfg
        shp = (c["n_layer"], c["n_seq"], c["n_embd"])
        return (np.ctypeslib.as_array(lib().wgo_gpt2_key_cache(self.h), shp),
                np.ctypeslib.as_array(lib().wgo_gpt2_value_cache(self.h), shp))

    def decode(self, prompt, n_gen: int, start_pos: int = 0) -> np.ndarray:
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        out = np.zeros(prompt.size - 1 + n_gen, dtype=np.uint32)
        lib().wgo_gpt2_decode(self.h, _p(prompt), prompt.size, n_gen, start_pos, _p(out))
        return out

    def __del__(self):
        if getattr(self, "h", None):
            lib().wgo_gpt2_free(self.h)
            self.h = None
