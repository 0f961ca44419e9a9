"""Generates tests/golden/dequant_golden.npz and tests/golden/gguf_dummy_expected.json.

Inputs: the deterministic block patterns that the reference's own `dequantization` test builds
(crates/wgml/src/ops/quantization.rs:79-222), restated here in numpy, plus seeded random blocks
with the value distributions of the GEMV microbench.  That test stores no outputs (it compares
the shader with `Block*::dequantize` at run time), so the expected values are produced by an
independent implementation of the same ggml formats: gguf-py's `quants.dequantize`, whose f32
operation order matches the Rust code for these formats.  Q8_K is absent from gguf-py; its
expected values are `d * qs` evaluated in numpy f32 (one rounding, nothing to disagree on).

The second output records what gguf-py's GGUFReader sees in the reference's
assets/gguf/dummy.gguf (the file of the `load_dummy_gguf` test, gguf.rs:715-722); a copy of that
11 KB fixture sits beside this script as ref_dummy.gguf.

Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import os

import numpy as np
from gguf import GGMLQuantizationType as T
from gguf import GGUFReader, quants

HERE = os.path.dirname(os.path.abspath(__file__))

F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q4_K, Q5_K, Q6_K, Q8_K = 0, 1, 2, 3, 6, 7, 8, 12, 13, 14, 15
GG = {Q4_0: T.Q4_0, Q4_1: T.Q4_1, Q5_0: T.Q5_0, Q5_1: T.Q5_1, Q8_0: T.Q8_0, Q4_K: T.Q4_K,
      Q5_K: T.Q5_K, Q6_K: T.Q6_K}
BLOCK_BYTES = {Q4_0: 18, Q4_1: 20, Q5_0: 22, Q5_1: 24, Q8_0: 34, Q4_K: 144, Q5_K: 176, Q6_K: 210,
               Q8_K: 292}


def f16_bits(v: float) -> bytes:
    return np.float16(v).tobytes()


def u16(v: int) -> bytes:
    return np.uint16(v).tobytes()


def sat_add_u8(base: int, k: int) -> int:
    return min(255, base + (k & 0xFF))


def sat_add_i8(base: int, k: int) -> int:
    k8 = ((k & 0xFF) ^ 0x80) - 0x80  # `k as i8`
    return max(-128, min(127, base + k8))


def reference_test_patterns() -> dict:
    """The inputs of ops/quantization.rs:79-222, as raw little-endian block bytes."""
    out = {}
    s1234, s5678 = f16_bits(1.234), f16_bits(5.678)
    # Q8_0 :79-84 -- 8 blocks, data[k] = i*16 - 128 + k
    out[Q8_0] = b"".join(s1234 + np.array([i * 16 - 128 + k for k in range(32)], np.int8).tobytes()
                         for i in range(8))
    ramp16 = lambda i: np.array([i * 16 + k for k in range(16)], np.uint8).tobytes()
    out[Q4_0] = b"".join(s1234 + ramp16(i) for i in range(16))                      # :88-93
    out[Q4_1] = b"".join(s1234 + u16(3) + ramp16(i) for i in range(16))             # :97-107
    qh = bytes([1, 100, 200, 250])
    out[Q5_0] = b"".join(s1234 + qh + ramp16(i) for i in range(16))                 # :111-120
    out[Q5_1] = b"".join(s1234 + u16(125) + qh + ramp16(i) for i in range(16))      # :124-134
    # Q8_K :138-148 -- d = 1.234f32, qs[k] = sat(i*8 - 127 + (k as i8)), bsums = 0
    out[Q8_K] = b"".join(np.float32(1.234).tobytes()
                         + np.array([sat_add_i8(i * 8 - 127, k) for k in range(256)], np.int8).tobytes()
                         + bytes(32) for i in range(16))
    # Q5_K :152-175 and Q4_K :179-201
    blocks5, blocks4 = [], []
    for i in range(16):
        scales = np.array([i * 16 + k for k in range(12)], np.uint8).tobytes()
        qs = np.array([sat_add_u8(i * 16, k) for k in range(128)], np.uint8).tobytes()
        qh5 = np.array([sat_add_u8(i * 16, k) for k in range(32)], np.uint8).tobytes()
        blocks5.append(s1234 + s5678 + scales + qh5 + qs)
        blocks4.append(s1234 + s5678 + scales + qs)
    out[Q5_K], out[Q4_K] = b"".join(blocks5), b"".join(blocks4)
    # Q6_K :205-221 -- d = raw bits 123
    blocks6 = []
    for i in range(16):
        scales = np.array([i * 8 - 127 + k for k in range(16)], np.int8).tobytes()
        ql = np.array([i * 8 + k for k in range(128)], np.uint8).tobytes()
        qh6 = np.array([i * 8 + k for k in range(64)], np.uint8).tobytes()
        blocks6.append(ql + qh6 + scales + u16(123))
    out[Q6_K] = b"".join(blocks6)
    return {k: np.frombuffer(v, np.uint8).copy() for k, v in out.items()}


def random_blocks(qtype: int, nblocks: int, rng: np.random.Generator) -> np.ndarray:
    """Uniform random codes; f16 scales = f16(|N(0,1)| * 0.01), as the GEMV microbench uses."""
    bb = BLOCK_BYTES[qtype]
    raw = rng.integers(0, 256, size=(nblocks, bb), dtype=np.uint8)

    def put_scale(col):
        s = (np.abs(rng.standard_normal(nblocks)) * 0.01).astype(np.float16)
        raw[:, col:col + 2] = s.view(np.uint8).reshape(nblocks, 2)

    if qtype in (Q4_0, Q5_0, Q8_0):
        put_scale(0)
    elif qtype in (Q4_1, Q5_1, Q4_K, Q5_K):
        put_scale(0)
        put_scale(2)
    elif qtype == Q6_K:
        put_scale(208)
    elif qtype == Q8_K:
        s = (np.abs(rng.standard_normal(nblocks)) * 0.01).astype(np.float32)
        raw[:, 0:4] = s.view(np.uint8).reshape(nblocks, 4)
    return raw.reshape(-1)


def expected(qtype: int, raw: np.ndarray) -> np.ndarray:
    if qtype == Q8_K:
        blocks = raw.reshape(-1, 292)
        d = blocks[:, 0:4].copy().view(np.float32)
        qs = blocks[:, 4:260].copy().view(np.int8).astype(np.float32)
        return (d * qs).astype(np.float32).reshape(-1)
    return quants.dequantize(raw, GG[qtype]).astype(np.float32).reshape(-1)


def main():
    arrays = {}
    rng = np.random.default_rng(20240607)
    for qtype, raw in reference_test_patterns().items():
        arrays[f"pattern_in_{qtype}"] = raw
        arrays[f"pattern_out_{qtype}"] = expected(qtype, raw)
    for qtype in BLOCK_BYTES:
        raw = random_blocks(qtype, 64, rng)
        arrays[f"random_in_{qtype}"] = raw
        arrays[f"random_out_{qtype}"] = expected(qtype, raw)
    # every f16 bit pattern, decoded by numpy (NaNs keep numpy's payload; compare as "both NaN")
    arrays["f16_all"] = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "dequant_golden.npz"), **arrays)

    path = os.path.join(HERE, "ref_dummy.gguf")
    r = GGUFReader(path)
    meta = {}
    for key, f in r.fields.items():
        if key.startswith("GGUF."):
            continue
        types = [t.name for t in f.types]
        if types[0] == "STRING":
            val = bytes(f.parts[-1]).decode()
        elif types[0] == "ARRAY":
            if types[1] == "STRING":
                val = [bytes(f.parts[i]).decode() for i in f.data]
            else:
                val = [f.parts[i][0].item() for i in f.data]
        else:
            val = f.parts[-1][0].item()
        meta[key] = {"types": types, "value": val}
    tensors = {t.name: {"type": int(t.tensor_type), "shape": [int(s) for s in t.shape],
                        "offset": int(t.data_offset), "first": float(t.data.ravel()[0]),
                        "sum": float(np.asarray(t.data, np.float64).sum())}
               for t in r.tensors}
    with open(os.path.join(HERE, "gguf_dummy_expected.json"), "w") as fh:
        json.dump({"version": 3, "metadata": meta, "tensors": tensors}, fh, indent=1, sort_keys=True)


if __name__ == "__main__":
    main()
