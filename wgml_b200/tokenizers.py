"""Tokenizers and the default chat template over the C ABI: the host mirror of `LlamaTokenizer`
(crates/wgml/src/models/llama2/tokenizer.rs), `Gpt2Tokenizer` (crates/wgml/src/models/gpt2/tokenizer.rs) and
`ChatTemplate` (crates/wgml-chat/src/chat_template.rs).  Host only: no device is needed."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import check
from .gguf import Gguf


def _text(fn, *args) -> str:
    n = C.c_size_t()
    check(fn(*args, None, 0, C.byref(n)))
    buf = C.create_string_buffer(n.value + 1)
    check(fn(*args, buf, n.value + 1, C.byref(n)))
    return buf.raw[:n.value].decode("utf-8", "replace")


class LlamaTokenizer:
    """LlamaTokenizer::from_gguf (tokenizer.rs:23-52)."""

    def __init__(self, gguf: Gguf):
        self._h = C.c_void_p()
        check(_lib.load().wgb_llama_tokenizer_from_gguf(gguf._h, C.byref(self._h)))
        lib = _lib.load()
        self.bos, self.eos, self.unk = (lib.wgb_llama_tokenizer_bos(self._h), lib.wgb_llama_tokenizer_eos(self._h),
                                        lib.wgb_llama_tokenizer_unk(self._h))

    @classmethod
    def from_gguf(cls, gguf: Gguf) -> "LlamaTokenizer":
        return cls(gguf)

    def encode(self, text: str, bos: bool, eos: bool) -> list[int]:
        raw = text.encode("utf-8")
        n = C.c_size_t()
        lib = _lib.load()
        check(lib.wgb_llama_tokenizer_encode(self._h, raw, len(raw), int(bos), int(eos), None, 0, C.byref(n)))
        out = np.zeros(max(n.value, 1), np.uint32)
        check(lib.wgb_llama_tokenizer_encode(self._h, raw, len(raw), int(bos), int(eos), out.ctypes.data, out.size, C.byref(n)))
        return [int(v) for v in out[:n.value]]

    def decode(self, prev_token: int, token: int) -> str:
        return _text(_lib.load().wgb_llama_tokenizer_decode, self._h, prev_token, token)

    def bos_str(self) -> str:
        return self.decode(0, self.bos)

    def eos_str(self) -> str:
        return self.decode(0, self.eos)

    def close(self):
        if self._h:
            _lib.load().wgb_llama_tokenizer_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Gpt2Tokenizer:
    """Gpt2Tokenizer::from_gguf (gpt2/tokenizer.rs:55-97)."""

    def __init__(self, gguf: Gguf):
        self._h = C.c_void_p()
        check(_lib.load().wgb_gpt2_tokenizer_from_gguf(gguf._h, C.byref(self._h)))
        lib = _lib.load()
        self.bos, self.eos = lib.wgb_gpt2_tokenizer_bos(self._h), lib.wgb_gpt2_tokenizer_eos(self._h)

    @classmethod
    def from_gguf(cls, gguf: Gguf) -> "Gpt2Tokenizer":
        return cls(gguf)

    def encode(self, text: str) -> list[int]:
        raw = text.encode("utf-8")
        n = C.c_size_t()
        lib = _lib.load()
        check(lib.wgb_gpt2_tokenizer_encode(self._h, raw, len(raw), None, 0, C.byref(n)))
        out = np.zeros(max(n.value, 1), np.uint32)
        check(lib.wgb_gpt2_tokenizer_encode(self._h, raw, len(raw), out.ctypes.data, out.size, C.byref(n)))
        return [int(v) for v in out[:n.value]]

    def decode(self, tokens) -> str:
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        return _text(_lib.load().wgb_gpt2_tokenizer_decode, self._h, t.ctypes.data, t.size)

    def close(self):
        if self._h:
            _lib.load().wgb_gpt2_tokenizer_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ChatTemplate:
    """ChatTemplate (chat_template.rs:5-40) for the default Llama-2 chat template."""

    @staticmethod
    def apply(messages: list[tuple[str, str]], bos: str, eos: str) -> str:
        """`messages`: (role, content) pairs, roles "system" (first only) / "user" / "assistant"."""
        n = len(messages)
        roles = (C.c_char_p * n)(*[r.encode() for r, _ in messages])
        contents = (C.c_char_p * n)(*[c.encode() for _, c in messages])
        return _text(_lib.load().wgb_chat_template_llama2, roles, contents, n, bos.encode(), eos.encode())
