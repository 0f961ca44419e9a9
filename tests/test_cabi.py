"""The C-ABI library builds, loads and exports every symbol include/wgml_b200.h declares; host-side
argument checks that need no GPU."""
import os
import re

import pytest

from conftest import ROOT
from wgml_b200 import _lib


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "wgml_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(wgb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) > 60
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"
    # and the Python binding types each of them
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)


def test_block_geometry():
    lib = _lib.load()
    expect = {0: (4, 1), 1: (2, 1), 2: (18, 32), 3: (20, 32), 6: (22, 32), 7: (24, 32), 8: (34, 32), 12: (144, 256),
              13: (176, 256), 14: (210, 256), 15: (292, 256), 9: (0, 0), 99: (0, 0)}
    for qt, (bb, bl) in expect.items():
        assert lib.wgb_block_bytes(qt) == bb and lib.wgb_block_len(qt) == bl


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from wgml_b200 import ops
    with pytest.raises(_lib.WgbError):
        ops.GemvQuant.from_device()
    with pytest.raises(_lib.WgbError):
        ops.require_device()


def test_argument_errors_are_statuses_not_aborts():
    lib = _lib.load()
    assert lib.wgb_dequantize(99, None, 1, None, None) != 0
    assert "null" in _lib.last_error() or "unsupported" in _lib.last_error()
    assert lib.wgb_rope(0, None, None, 2, None, 2, None) == _lib.ERR_INVALID
    assert lib.wgb_gguf_open(b"/nonexistent/file.gguf", None) == _lib.ERR_INVALID  # null out pointer
