"""GGUF parser: the reference's own fixture (assets/gguf/dummy.gguf, copied as golden/ref_dummy.gguf)
against what gguf-py's reader sees in it, files written by gguf-py's writer with quantised tensors,
and malformed input."""
import ctypes as C
import json
import os

import numpy as np
import pytest

from conftest import ROOT
from wgml_b200 import _lib
from wgml_b200.gguf import Gguf
from wgml_b200._lib import WgbError

GOLD = os.path.join(ROOT, "tests", "golden")


def test_reference_dummy_gguf_matches_gguf_py():
    exp = json.load(open(os.path.join(GOLD, "gguf_dummy_expected.json")))
    g = Gguf.open(os.path.join(GOLD, "ref_dummy.gguf"))
    assert g.version == exp["version"] == 3
    assert g.alignment == 32
    assert set(g.metadata) == set(exp["metadata"])
    for key, e in exp["metadata"].items():
        got, want = g.metadata[key], e["value"]
        if isinstance(want, float) or (isinstance(want, list) and want and isinstance(want[0], float)):
            assert np.allclose(got, want, rtol=0, atol=0), key
        else:
            assert got == want, key
        kinds = {"UINT8": "U8", "INT8": "I8", "UINT16": "U16", "INT16": "I16", "UINT32": "U32", "INT32": "I32",
                 "FLOAT32": "F32", "UINT64": "U64", "INT64": "I64", "FLOAT64": "F64", "BOOL": "Bool", "STRING": "String",
                 "ARRAY": "Array"}
        assert g.meta_type(key) == kinds[e["types"][0]]
    assert set(g.tensors) == set(exp["tensors"])
    for name, e in exp["tensors"].items():
        t = g.tensors[name]
        assert t.type == e["type"] == 0
        assert t.dimensions[: len(e["shape"])] == e["shape"][::-1] or sorted(t.dimensions[: len(e["shape"])]) == sorted(e["shape"])
        assert t.offset == e["offset"]
        data = t.as_f32()
        assert data.size == int(np.prod(e["shape"]))
        assert data[0] == e["first"] and float(data.astype(np.float64).sum()) == e["sum"]


def _write(path, arch="llama", align=None, tensors=None, extra=None):
    import gguf
    w = gguf.GGUFWriter(path, arch)
    if align:
        w.add_custom_alignment(align)
    for k, v in (extra or {}).items():
        if isinstance(v, int):
            w.add_uint32(k, v)
        elif isinstance(v, float):
            w.add_float32(k, v)
        elif isinstance(v, list):
            w.add_array(k, v)
        else:
            w.add_string(k, v)
    for name, (arr, rtype) in (tensors or {}).items():
        w.add_tensor(name, arr, raw_dtype=rtype)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def test_quantised_tensors_and_alignment(tmp_path):
    import gguf
    from wgml_b200 import synth
    rng = np.random.default_rng(5)
    q4 = synth.quant_blocks(synth.Q4_K, 8, rng).reshape(2, 4 * 144)
    q6 = synth.quant_blocks(synth.Q6_K, 4, rng).reshape(2, 2 * 210)
    q8 = synth.quant_blocks(synth.Q8_0, 16, rng).reshape(4, 4 * 34)
    f = rng.standard_normal((3, 5)).astype(np.float32)
    path = str(tmp_path / "q.gguf")
    _write(path, align=64, extra={"llama.block_count": 2, "general.name": "t"},
           tensors={"a.q4": (q4, gguf.GGMLQuantizationType.Q4_K), "b.q6": (q6, gguf.GGMLQuantizationType.Q6_K),
                    "c.q8": (q8, gguf.GGMLQuantizationType.Q8_0), "d.f32": (f, None)})
    g = Gguf.open(path)
    assert g.alignment == 64 and g.metadata["general.alignment"] == 64
    assert g.metadata["llama.block_count"] == 2 and g.metadata["general.name"] == "t"
    assert g.tensors["a.q4"].type == 12 and np.array_equal(g.tensors["a.q4"].data(), q4.reshape(-1))
    assert g.tensors["b.q6"].type == 14 and np.array_equal(g.tensors["b.q6"].data(), q6.reshape(-1))
    assert g.tensors["c.q8"].type == 8 and np.array_equal(g.tensors["c.q8"].data(), q8.reshape(-1))
    assert np.array_equal(g.tensors["d.f32"].as_f32(), f.reshape(-1))
    assert g.tensors["a.q4"].dimensions[:2] == [1024, 2]  # GGUF stores the contiguous dimension first
    assert all(t.offset % 64 == 0 for t in g.tensors.values())
    # from_bytes sees the same thing as the mapping
    g2 = Gguf.from_bytes(open(path, "rb").read())
    assert set(g2.tensors) == set(g.tensors) and g2.metadata == g.metadata


def test_llama_config_from_gguf(tmp_path):
    from wgml_b200.models import Llama2Config, LlamaModelType
    path = str(tmp_path / "cfg.gguf")
    _write(path, extra={"llama.embedding_length": 288, "llama.feed_forward_length": 768, "llama.block_count": 6,
                        "llama.attention.head_count": 6, "llama.attention.head_count_kv": 3, "llama.context_length": 256,
                        "tokenizer.ggml.tokens": ["a", "b", "c"]})
    cfg = Llama2Config.from_gguf(Gguf.open(path))
    assert (cfg.dim, cfg.hidden_dim, cfg.n_layers, cfg.n_q_heads, cfg.n_kv_heads, cfg.vocab_size, cfg.seq_len) == \
        (288, 768, 6, 6, 3, 3, 256)
    # defaults of cpu.rs:98-107 when the keys are absent
    assert cfg.rope_base_freq == 10000.0 and abs(cfg.rms_norm_eps - 1e-6) < 1e-12
    with pytest.raises(WgbError) as e:
        Llama2Config.from_gguf(Gguf.open(path), LlamaModelType.Qwen2)  # looks for qwen2.* keys
    assert e.value.status == _lib.ERR_NOT_FOUND


def test_malformed_files_are_errors(tmp_path):
    good = open(os.path.join(GOLD, "ref_dummy.gguf"), "rb").read()
    with pytest.raises(WgbError) as e:
        Gguf.from_bytes(b"GGML" + good[4:])
    assert e.value.status == _lib.ERR_PARSE and "magic" in e.value.message
    for cut in (3, 10, 24, 40, 200, 1000, 1215, len(good) - 1):
        with pytest.raises(WgbError) as e:
            Gguf.from_bytes(good[:cut])
        assert e.value.status == _lib.ERR_PARSE, cut
    # unknown metadata value type (gguf.rs:382) and unknown tensor type (gguf.rs:103)
    bad = bytearray(good)
    key_len = int.from_bytes(good[24:32], "little")
    bad[32 + key_len:36 + key_len] = (13).to_bytes(4, "little")
    with pytest.raises(WgbError) as e:
        Gguf.from_bytes(bytes(bad))
    assert e.value.status == _lib.ERR_UNSUPPORTED
    with pytest.raises(WgbError) as e:
        Gguf.open(str(tmp_path / "missing.gguf"))
    assert e.value.status == _lib.ERR_NOT_FOUND


def test_big_endian_magic_is_accepted_like_the_reference():
    good = bytearray(open(os.path.join(GOLD, "ref_dummy.gguf"), "rb").read())
    good[0:4] = (0x47475546).to_bytes(4, "little")  # GGUF_FILE_MAGIC_BE, gguf.rs:20,477
    assert Gguf.from_bytes(bytes(good)).version == 3


def test_mutated_files_parse_or_fail_cleanly():
    """Random byte, word and length mutations of a valid file: every one either parses -- and then every tensor's
    bytes and every metadata value can be read -- or is refused with a status; none may crash the process.  Strings that
    are not UTF-8 come out with replacement characters, as the reference reads them (gguf.rs:660, from_utf8_lossy)."""
    import random
    good = open(os.path.join(GOLD, "ref_dummy.gguf"), "rb").read()
    rng = random.Random(2024)
    parsed = refused = 0
    for _ in range(1500):
        b = bytearray(good)
        mode = rng.randrange(4)
        if mode == 0:
            for _ in range(rng.randint(1, 4)):
                b[rng.randrange(len(b))] = rng.randrange(256)
        elif mode == 1:
            p = rng.randrange(0, min(len(b) - 8, 1400))
            b[p:p + 8] = rng.choice([0, 1, 0xFF, 0xFFFF, 0xFFFFFFFF, 2**63, 2**64 - 1, rng.getrandbits(64)]).to_bytes(8, "little")
        elif mode == 2:
            b = b[:rng.randrange(len(b))]
        else:
            p = rng.randrange(0, min(len(b) - 4, 1400))
            b[p:p + 4] = rng.getrandbits(32).to_bytes(4, "little")
        try:
            g = Gguf.from_bytes(bytes(b))
        except WgbError as e:
            assert e.status in (_lib.ERR_PARSE, _lib.ERR_UNSUPPORTED, _lib.ERR_INVALID), e.status
            refused += 1
            continue
        for t in g.tensors.values():
            d = t.data()
            assert d.size == t.n_bytes or d.size == 0
            if d.size:
                int(d[0]) + int(d[-1])
        repr(g.metadata)
        g.close()
        parsed += 1
    assert parsed > 100 and refused > 100
    # a tensor name that is not UTF-8
    bad = bytearray(good)
    bad[good.index(b"tensor")] = 0xFF
    g = Gguf.from_bytes(bytes(bad))
    assert any("\ufffd" in n for n in list(g.tensors) + list(g.metadata))
