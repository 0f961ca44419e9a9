"""`Gguf` (crates/wgml/src/gguf.rs:317-322) over the C parser: metadata and tensor directory."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import GgufTensorC, WgbError, check

META_TYPES = ["U8", "I8", "U16", "I16", "U32", "I32", "F32", "Bool", "String", "Array", "U64", "I64", "F64"]
_INT = {0, 1, 2, 3, 4, 5, 10, 11}
_SIGNED = {1, 3, 5, 11}
_FLOAT = {6, 12}


class GgufTensor:
    """GgufTensor (gguf.rs:297-315): dimensions, ggml type and a zero-copy view of the bytes."""

    def __init__(self, info: GgufTensorC, owner):
        self.name = info.name.decode("utf-8", "replace")   # lossy, as the reference reads strings (gguf.rs:660)
        self.n_dims = info.n_dims
        self.dimensions = [int(d) for d in info.dims]
        self.type = int(info.type)
        self.offset = int(info.offset)
        self.n_bytes = int(info.n_bytes)
        self._ptr = info.data
        self._owner = owner

    def data(self) -> np.ndarray:
        """The raw bytes (empty for types the reference leaves unread)."""
        if not self._ptr or not self.n_bytes:
            return np.zeros(0, np.uint8)
        buf = (C.c_uint8 * self.n_bytes).from_address(self._ptr)
        a = np.frombuffer(buf, dtype=np.uint8)
        a.flags.writeable = False
        return a

    def as_f32(self) -> np.ndarray:
        if self.type != 0:
            raise WgbError(_lib.ERR_INVALID, f"tensor '{self.name}' is not f32")
        return self.data().view(np.float32)


class Gguf:
    """Parsed GGUF file.  `Gguf.open(path)` maps the file; `Gguf.from_bytes(b)` parses a buffer."""

    def __init__(self, handle, keep=None):
        self._h = handle
        self._keep = keep
        lib = _lib.load()
        self.version = lib.wgb_gguf_version(handle)
        self.alignment = lib.wgb_gguf_alignment(handle)
        self.metadata = {}
        for i in range(lib.wgb_gguf_metadata_count(handle)):
            self.metadata[lib.wgb_gguf_meta_key(handle, i).decode("utf-8", "replace")] = self._value(i)
        self.tensors = {}
        info = GgufTensorC()
        for i in range(lib.wgb_gguf_tensor_count(handle)):
            check(lib.wgb_gguf_tensor_info(handle, i, C.byref(info)))
            t = GgufTensor(info, self)
            self.tensors[t.name] = t

    @classmethod
    def open(cls, path: str) -> "Gguf":
        h = C.c_void_p()
        check(_lib.load().wgb_gguf_open(path.encode(), C.byref(h)))
        return cls(h)

    @classmethod
    def from_bytes(cls, data) -> "Gguf":
        buf = np.frombuffer(data, dtype=np.uint8)
        h = C.c_void_p()
        check(_lib.load().wgb_gguf_from_bytes(buf.ctypes.data, buf.size, C.byref(h)))
        return cls(h, keep=buf)

    def _value(self, i):
        lib = _lib.load()
        ty, et, ln = C.c_int(), C.c_int(), C.c_uint64()
        check(lib.wgb_gguf_meta_type(self._h, i, C.byref(ty), C.byref(et), C.byref(ln)))
        t = ty.value

        def scalar(kind, getter_u, getter_i, getter_f, *idx):
            if kind in _FLOAT:
                v = C.c_double()
                check(getter_f(self._h, i, *idx, C.byref(v)))
                return float(np.float32(v.value)) if kind == 6 else v.value
            if kind in _SIGNED:
                v = C.c_int64()
                check(getter_i(self._h, i, *idx, C.byref(v)))
                return v.value
            v = C.c_uint64()
            check(getter_u(self._h, i, *idx, C.byref(v)))
            return bool(v.value) if kind == 7 else v.value

        if t == 8:
            p, n = C.c_void_p(), C.c_uint64()
            check(lib.wgb_gguf_meta_str(self._h, i, C.byref(p), C.byref(n)))
            return C.string_at(p.value, n.value).decode("utf-8", "replace") if n.value else ""
        if t == 9:
            e = et.value
            if e == 8:
                out = []
                p, n = C.c_void_p(), C.c_uint64()
                for j in range(ln.value):
                    check(lib.wgb_gguf_meta_arr_str(self._h, i, j, C.byref(p), C.byref(n)))
                    out.append(C.string_at(p.value, n.value).decode("utf-8", "replace") if n.value else "")
                return out
            if e == 9:
                return [None] * ln.value  # nested arrays: length only
            return [scalar(e, lib.wgb_gguf_meta_arr_u64, lib.wgb_gguf_meta_arr_i64, lib.wgb_gguf_meta_arr_f64, j)
                    for j in range(ln.value)]
        return scalar(t, lib.wgb_gguf_meta_u64, lib.wgb_gguf_meta_i64, lib.wgb_gguf_meta_f64)

    def meta_type(self, key: str) -> str:
        lib = _lib.load()
        i = lib.wgb_gguf_meta_find(self._h, key.encode())
        if i < 0:
            raise KeyError(key)
        ty = C.c_int()
        check(lib.wgb_gguf_meta_type(self._h, i, C.byref(ty), None, None))
        return META_TYPES[ty.value]

    def close(self):
        if self._h is not None and self._h.value:
            _lib.load().wgb_gguf_close(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
