"""GGUF -> device load throughput of the Llama loader (`wgb_llama2_load_gguf`).

    python -m wgml_b200.load_bench [--workload llama2-7b] [--layers N] [--dir /tmp] [--tp-size T --tp-rank R]

Writes a synthetic GGUF of the named configuration (random blocks, the tensor names and metadata keys of
Llama2Weights::from_gguf, crates/wgml/src/models/llama2/transformer.rs:151-268), maps it, loads it and prints
one JSON line: file bytes, bytes uploaded (a tensor-parallel rank uploads its slices only), seconds and GB/s
for a cold-ish first load and a second load with the file in the page cache.  The reference reads every tensor
eagerly, element by element, into host vectors before anything reaches the GPU
(crates/wgml/src/gguf.rs:539-620, 671-681); here the bytes go from the mapping through pinned buffers straight
to their place in HBM, repacked on the device where the format needs it.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import numpy as np

from . import synth
from .gguf import Gguf
from .models import Llama2, LlamaModelType

GG = {synth.Q4_K: "Q4_K", synth.Q6_K: "Q6_K", synth.Q8_0: "Q8_0", synth.F32: "F32"}


def write_gguf(path: str, cfg: dict, seed: int = 0) -> int:
    import gguf
    w = gguf.GGUFWriter(path, "llama")
    w.add_uint32("llama.embedding_length", cfg["dim"])
    w.add_uint32("llama.feed_forward_length", cfg["hidden_dim"])
    w.add_uint32("llama.block_count", cfg["n_layers"])
    w.add_uint32("llama.attention.head_count", cfg["n_q_heads"])
    w.add_uint32("llama.attention.head_count_kv", cfg["n_kv_heads"])
    w.add_uint32("llama.context_length", cfg["seq_len"])
    w.add_float32("llama.attention.layer_norm_rms_epsilon", cfg["rms_norm_eps"])
    w.add_array("tokenizer.ggml.tokens", [f"t{i}" for i in range(cfg["vocab_size"])])
    dim, hid, vocab = cfg["dim"], cfg["hidden_dim"], cfg["vocab_size"]
    kv = dim * cfg["n_kv_heads"] // cfg["n_q_heads"]
    shapes = {"attn_q": (dim, dim), "attn_k": (kv, dim), "attn_v": (kv, dim), "attn_output": (dim, dim),
              "ffn_gate": (hid, dim), "ffn_up": (hid, dim), "ffn_down": (dim, hid), "token_embd": (vocab, dim), "output": (vocab, dim)}
    keep = []
    for l in range(cfg["n_layers"]):
        t = synth.llama_tensors(cfg, seed, layers=[l], model_tensors=(l == 0))
        for name, (qt, arr) in t.items():
            if qt == synth.F32:
                a = np.asarray(arr, np.float32)
                keep.append(a)
                w.add_tensor(name, a)
            else:
                r, c = shapes[name.split(".")[-2]]
                a = np.asarray(arr).reshape(r, c // synth.BLOCK_LEN[qt] * synth.BLOCK_BYTES[qt])
                keep.append(a)
                w.add_tensor(name, a, raw_dtype=getattr(gguf.GGMLQuantizationType, GG[qt]))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return os.path.getsize(path)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="llama2-7b", choices=["llama2-7b", "llama2-70b", "tiny-llama"])
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--dir", default="/tmp")
    ap.add_argument("--tp-size", type=int, default=1)
    ap.add_argument("--tp-rank", type=int, default=0)
    a = ap.parse_args()
    cfg = dict(synth.CONFIGS[a.workload], seq_len=64)
    if a.layers:
        cfg["n_layers"] = a.layers
    path = os.path.join(a.dir, f"wgml_b200_{a.workload}_{cfg['n_layers']}l.gguf")
    t0 = time.time()
    size = write_gguf(path, cfg)
    t_write = time.time() - t0
    runs = []
    for _ in range(2):
        g = Gguf.open(path)
        t0 = time.time()
        m = Llama2.from_gguf(g, LlamaModelType.Llama, a.tp_rank, a.tp_size)
        wall = time.time() - t0
        b, s = m.load_stats()
        runs.append({"uploaded_bytes": b, "upload_seconds": s, "gb_per_s": b / s / 1e9 if s > 0 else None, "wall_seconds": wall})
        m.close()
    os.remove(path)
    print(json.dumps({"workload": a.workload, "layers": cfg["n_layers"], "file_bytes": size, "write_seconds": t_write,
                      "tp": [a.tp_rank, a.tp_size], "loads": runs}))


if __name__ == "__main__":
    main()
