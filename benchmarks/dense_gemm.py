"""Dense GEMM benchmark (one B200): the model's dense projections on the hand-written tcgen05 GEMM (the grouped
kernel with one segment) against the library GEMM (``torch.matmul``, cuBLAS), forward, input gradient and weight
gradient, timed with CUDA events after warm-up with a buffer larger than L2 written between iterations.

Shapes (tokens x in -> out): Qwen3-30B-A3B qkv 8192 x 2048 -> 5120 and output 8192 x 4096 -> 2048, the vocabulary
projection 8192 x 2048 -> 151936, and the DeepSeek-V3 proxy's dense feed-forward 4096 x 7168 -> 36864.

    python benchmarks/dense_gemm.py [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

SHAPES = [("qkv", 8192, 2048, 5120), ("attn out", 8192, 4096, 2048), ("vocab", 8192, 2048, 151936),
          ("dense ffn up", 4096, 7168, 36864), ("mla kv_a", 4096, 7168, 576)]


def timeit(fn, flush, iters=8, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default="")
    ap.add_argument("--iters", type=int, default=8)
    args = ap.parse_args(argv)
    from system_lab_b200.ops import cuda as cops
    peaks = {}
    pf = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pf):
        peaks = json.load(open(pf))
    peak = float(peaks.get("bf16_tflops", 1590.0))
    basis = "of measured" if peaks else "of fallback"
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    for name, r, k, n in SHAPES:
        torch.manual_seed(0)
        x = torch.randn(r, k, device=dev, dtype=torch.bfloat16)
        w = (0.02 * torch.randn(n, k, device=dev)).to(torch.bfloat16)
        g = torch.randn(r, n, device=dev, dtype=torch.bfloat16)
        off, cnt = cops._dense_segments(dev, r)
        y, dx, dw = torch.empty(r, n, device=dev, dtype=torch.bfloat16), torch.empty_like(x), torch.empty_like(w)
        flops = 2.0 * r * k * n
        ops = {
            "fwd": (lambda: cops.grouped_gemm_raw(0, x, w, off, cnt, n, k, out=y, block_n=cops._pick_bn(n)),
                    lambda: torch.matmul(x, w.t(), out=y)),
            "dgrad": (lambda: cops.grouped_gemm_raw(1, g, w, off, cnt, n, k, out=dx, block_n=cops._pick_bn(k)),
                      lambda: torch.matmul(g, w, out=dx)),
            "wgrad": (lambda: cops.grouped_gemm_raw(2, g, x, off, cnt, n, k, out=dw, block_n=cops._pick_bn(k)),
                      lambda: torch.matmul(g.t(), x, out=dw)),
        }
        for op, (own, lib) in ops.items():
            t_own = timeit(own, flush, args.iters)
            t_lib = timeit(lib, flush, args.iters)
            cops.check_status()
            rec = {"shape": name, "rows": r, "in": k, "out": n, "op": op, "own_ms": t_own, "library_ms": t_lib,
                   "own_tflops": flops / t_own / 1e9, "library_tflops": flops / t_lib / 1e9,
                   "own_frac_of_peak": flops / t_own / 1e9 / peak, "peak_basis": basis}
            rows.append(rec)
            print(f"{name:13s} {op:6s} own {t_own:7.3f} ms {rec['own_tflops']:7.0f} TFLOP/s ({rec['own_frac_of_peak']:.2f} "
                  f"{basis})   library {t_lib:7.3f} ms {rec['library_tflops']:7.0f} TFLOP/s", flush=True)
        del x, w, g, y, dx, dw
        torch.cuda.empty_cache()
    if args.json:
        with open(args.json, "w") as f:
            json.dump({"peak_tflops": peak, "peak_basis": basis, "rows": rows}, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
