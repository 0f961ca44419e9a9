"""Quantised matrix-vector microbenchmark through the C ABI (`wgb_gemv_quant`).

    python -m wgml_b200.gemv_bench [--qtypes q4_k,q6_k,q8_0] [--shapes 4096x4096,...] [--reps 100]
                                   [--eager N] [--json] [--tensor] [--batched N]

The shapes and value distributions are those of wgml-bench's GEMV sweep restricted to the transformer
shapes of a 7B model (crates/wgml-bench/src/main.rs:186-248 times `GemvQuant::dispatch` on random block
bits): codes uniform, f16 scales |N(0,1)| * 0.01, x ~ N(0,1).

Timing: every launch reads a different copy of the matrix (enough copies to exceed the 126 MB L2 several
times over), so each one streams from HBM.  `--reps` launches are captured in one CUDA graph and the graph
is replayed three times between CUDA events.  The figure printed is algorithmic bytes
(rows * cols * bytes-per-weight of the GGUF format + 4 * cols + 4 * rows) per second.
`--eager N` instead issues N plain launches and exits; it exists for profilers, which want few launches.
`--tensor` times the tcgen05 path (`wgb_gemv_q4k_tiles`, Q4_K, up to 4096 columns) instead of `wgb_gemv_quant`.
`--batched N` times the batched tcgen05 products of the prompt prefill (`wgb_gemm_q4k_tiles` / `_q6k_` / `_q80_`, N = 1..8 input
vectors per launch: image of the inputs, product, sum of the column slices).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

import numpy as np
import torch

from . import _lib, synth

QT = {"q8_0": synth.Q8_0, "q4_k": synth.Q4_K, "q6_k": synth.Q6_K, "f32": synth.F32}
BPE = {synth.F32: 4.0, synth.Q8_0: 34 / 32, synth.Q4_K: 144 / 256, synth.Q6_K: 210 / 256}


def run(qtypes, shapes, reps, eager, peak_gbs, tensor=False, batched=0):
    lib = _lib.load()
    out = []
    for name in qtypes:
        qt = QT[name]
        for (n, k) in shapes:
            if tensor and (qt != synth.Q4_K or k > 4096 or n % 128):
                continue
            if batched and (qt not in (synth.Q4_K, synth.Q6_K, synth.Q8_0) or k % 256 or n % 128):
                continue
            tiles = {synth.Q4_K: ("wgb_q4k_tiles_create", "wgb_gemm_q4k_tiles", "wgb_q4k_tiles_destroy"),
                     synth.Q6_K: ("wgb_q6k_tiles_create", "wgb_gemm_q6k_tiles", "wgb_q6k_tiles_destroy"),
                     synth.Q8_0: ("wgb_q80_tiles_create", "wgb_gemm_q80_tiles", "wgb_q80_tiles_destroy")}.get(qt)
            nbytes = n * k * BPE[qt]
            ncopy = max(2, int(np.ceil(400e6 / nbytes)))
            rng = np.random.default_rng(1)
            if qt == synth.F32:
                raw = rng.standard_normal(n * k).astype(np.float32)
            else:
                raw = synth.quant_blocks(qt, n * k // synth.BLOCK_LEN[qt], rng)
            mats = []
            for _ in range(ncopy):
                h = C.c_void_p()
                if batched:
                    _lib.check(getattr(lib, tiles[0])(raw.ctypes.data, n, k, None, C.byref(h)))
                elif tensor:
                    _lib.check(lib.wgb_q4k_tiles_create(raw.ctypes.data, n, k, None, C.byref(h)))
                else:
                    _lib.check(lib.wgb_quant_matrix_create(qt, raw.ctypes.data, n, k, None, C.byref(h)))
                mats.append(h)
            gemv = lib.wgb_gemv_q4k_tiles if tensor else lib.wgb_gemv_quant
            x = torch.randn(max(batched, 1), k, device="cuda")
            y = torch.zeros(max(batched, 1), n, device="cuda")
            if batched:
                def gemv(h, xp, yp, stream, _f=getattr(lib, tiles[1])):
                    return _f(h, xp, batched, yp, stream)
            st = torch.cuda.current_stream().cuda_stream
            if eager:
                for it in range(eager):
                    _lib.check(gemv(mats[it % ncopy], x.data_ptr(), y.data_ptr(), st))
                torch.cuda.synchronize()
                out.append({"qtype": name, "rows": n, "cols": k, "eager_launches": eager})
            else:
                for it in range(max(20, ncopy)):   # also the first call on every copy (it may allocate)
                    _lib.check(gemv(mats[it % ncopy], x.data_ptr(), y.data_ptr(), st))
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    st2 = torch.cuda.current_stream().cuda_stream
                    for it in range(reps):
                        _lib.check(gemv(mats[it % ncopy], x.data_ptr(), y.data_ptr(), st2))
                g.replay()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(3):
                    g.replay()
                e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / (3 * reps)
                alg = nbytes + 4 * k + 4 * n
                out.append({"qtype": name + ("/tcgen05" if tensor else f"/tcgen05 x{batched}" if batched else ""), "rows": n, "cols": k, "us": us, "bytes": alg, "gbs": alg / us / 1e3,
                            "frac_of_measured_peak": alg / us / 1e3 / peak_gbs, "copies": ncopy})
            for h in mats:
                (getattr(lib, tiles[2]) if batched else lib.wgb_q4k_tiles_destroy if tensor else lib.wgb_quant_matrix_destroy)(h)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--qtypes", default="q8_0,q4_k,q6_k")
    ap.add_argument("--shapes", default="4096x4096,11008x4096,4096x11008,32000x4096")
    ap.add_argument("--reps", type=int, default=100)
    ap.add_argument("--eager", type=int, default=0)
    ap.add_argument("--peak-gbs", type=float, default=6550.7, help="HBM copy bandwidth the fraction is taken of")
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--tensor", action="store_true", help="time the tcgen05 path (Q4_K, up to 4096 columns)")
    ap.add_argument("--batched", type=int, default=0, help="time the batched tcgen05 product with this many input vectors (1..8)")
    a = ap.parse_args()
    shapes = [tuple(int(v) for v in s.split("x")) for s in a.shapes.split(",")]
    res = run(a.qtypes.split(","), shapes, a.reps, a.eager, a.peak_gbs, a.tensor, a.batched)
    if a.json:
        print(json.dumps(res))
        return
    for r in res:
        if "us" in r:
            print(f"{r['qtype']:12s} {r['rows']:6d}x{r['cols']:<6d} {r['us']:8.2f} us  {r['gbs']:8.1f} GB/s  "
                  f"{100 * r['frac_of_measured_peak']:5.1f}% of {a.peak_gbs:.0f} GB/s")
        else:
            print(f"{r['qtype']:12s} {r['rows']:6d}x{r['cols']:<6d} {r['eager_launches']} eager launches")


if __name__ == "__main__":
    main()
