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


def test_header_is_plain_c_and_links_from_c(tmp_path):
    """The boundary is a C ABI: the header compiles as pedantic C11 and as C++, and a C program with no other
    dependency links against the library and calls into it (host-only entry points: no device needed)."""
    import shutil
    import subprocess
    if not shutil.which("gcc"):
        pytest.skip("no C compiler")
    src = tmp_path / "user.c"
    src.write_text('#include <stdio.h>\n#include <string.h>\n#include "wgml_b200.h"\n'
                   "int main(void) {\n"
                   "    wgb_gguf *g = NULL;\n"
                   '    if (wgb_block_bytes(12) != 144 || wgb_block_len(12) != 256) return 1;\n'
                   '    if (wgb_gguf_from_bytes("GGML", 4, &g) == WGB_OK) return 2;\n'
                   '    if (!strlen(wgb_last_error()) || !strlen(wgb_version())) return 3;\n'
                   '    puts(wgb_version());\n'
                   "    return 0;\n}\n")
    inc = os.path.join(ROOT, "include")
    libdir = os.path.join(ROOT, "wgml_b200")
    for cc, std, lang in (("gcc", "-std=c11", "c"), ("g++", "-std=c++17", "c++")):
        if shutil.which(cc):
            r = subprocess.run([cc, std, "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", "-x", lang, "-I", inc, str(src)],
                               capture_output=True, text=True)
            assert r.returncode == 0, r.stderr
    exe = tmp_path / "user"
    r = subprocess.run(["gcc", "-std=c11", "-I", inc, str(src), "-o", str(exe), "-L", libdir, "-lwgml_b200", f"-Wl,-rpath,{libdir}"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.strip(), (r.returncode, r.stdout, r.stderr)


def _split_params(s: str):
    s = s.strip()
    if not s or s == "void":
        return []
    return [p.strip() for p in s.split(",")]


def test_binding_excerpt_in_the_integration_notes_matches_the_header():
    """Every `pub fn wgb_*` of the Rust excerpt names a declared entry point with the same number of parameters and the
    same parameter names (the excerpt is what a maintainer would copy)."""
    header = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "wgml_b200.h")).read(), flags=re.S)
    c_decls = {m.group(1): _split_params(m.group(2))
               for m in re.finditer(r"\b(wgb_[a-z0-9_]+)\s*\(([^()]*)\)\s*;", header)}
    notes = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    rust = re.findall(r"pub fn (wgb_[a-z0-9_]+)\(([^()]*)\)", notes)
    assert len(rust) >= 10
    for name, params in rust:
        assert name in c_decls, f"{name} is in the binding excerpt but not in the header"
        r = [p.split(":")[0].strip() for p in _split_params(params)]
        c = [re.findall(r"[A-Za-z_][A-Za-z0-9_]*", p)[-1] for p in c_decls[name]]
        assert r == c, f"{name}: Rust excerpt has {r}, the header {c}"
