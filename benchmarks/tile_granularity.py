"""Tile-granularity study of the grouped GEMM (one B200): one [M, K] x [K, N] product cut along M into 1 ... M/128
independent segments, all run by ONE persistent launch of the grouped kernel, against the same segments launched one
library GEMM at a time.

    python benchmarks/tile_granularity.py [--m 8192] [--k 7168] [--n 4096] [--max-segments 64] [--iters 10] [--json out.json]

Every segment multiplies its own copy of the weight matrix (as experts do: the kernel addresses weights by segment),
in the grouped launch and in the library loop alike, so the weight traffic grows with the number of segments for both.

Question (from the reference's overlap study): how small can the unit of work be made, so that a consumer can start on
the first rows while later rows are still arriving, before splitting costs throughput?  With one launch per tile the
reference measured a floor of 0.185 ms per tile below M <= 1024 (``notes/2026-04/2026-04-14_tile_overlap_analysis.md:
147-158``) and 524 TFLOP/s for its tile GEMM against 1000-1369 for the library (``:136-141,433-438``).  A persistent
kernel pays the launch once: the table shows how the time of the grouped kernel and of per-segment library launches
moves with the number of segments.

Timing: CUDA events on the launching stream, 3 warm-ups, median, a 256 MB write between iterations (cold L2).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def time_cuda(fn, flush, iters, warmup=3):
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
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--k", type=int, default=7168)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--max-segments", type=int, default=64, help="weight copies held at once (64 x N x K bf16)")
    ap.add_argument("--json", default="")
    args = ap.parse_args(argv)
    from system_lab_b200.ops import cuda as cops
    dev = torch.device("cuda")
    m, k, n = args.m, args.k, args.n
    if m % 128 or k % 64 or n % 128:
        raise SystemExit("m % 128, k % 64 and n % 128 must be 0")
    a = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
    w1 = (0.02 * torch.randn(n, k, device=dev)).to(torch.bfloat16)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    flops = 2.0 * m * k * n
    peaks = {}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    peak = peaks.get("bf16_tflops", 1590.0)
    rows = []
    print(f"[{m}, {k}] x [{k}, {n}] bf16, {flops / 1e12:.3f} TFLOP; peak {peak:.0f} TFLOP/s "
          f"({'measured' if peaks else 'fallback'})")
    print(f"{'segments':>9} {'rows/seg':>9} {'grouped ms':>11} {'TFLOP/s':>9} {'of peak':>8} {'per-seg launches ms':>20} {'TFLOP/s':>9}")
    segs = 1
    max_segs = min(m // 128, args.max_segments)
    while segs <= max_segs:
        per = m // segs
        w = w1.unsqueeze(0).expand(segs, n, k).contiguous()             # one weight copy per segment
        offsets = torch.arange(segs, device=dev, dtype=torch.int32) * per
        counts = torch.full((segs,), per, device=dev, dtype=torch.int32)
        out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        t_g = time_cuda(lambda: cops.grouped_gemm_raw(0, a, w, offsets, counts, n, k, out=out), flush, args.iters)

        def loop():
            for s in range(segs):
                torch.matmul(a[s * per:(s + 1) * per], w[s].t())
        t_l = time_cuda(loop, flush, args.iters)
        del w
        rows.append({"segments": segs, "rows_per_segment": per, "grouped_ms": t_g, "library_loop_ms": t_l,
                     "grouped_tflops": flops / (t_g * 1e9), "library_tflops": flops / (t_l * 1e9)})
        print(f"{segs:9d} {per:9d} {t_g:11.3f} {flops / (t_g * 1e9):9.0f} {flops / (t_g * 1e9) / peak:8.2f} "
              f"{t_l:20.3f} {flops / (t_l * 1e9):9.0f}")
        segs *= 2
    cops.check_status()
    if args.json:
        os.makedirs(os.path.dirname(args.json) or ".", exist_ok=True)
        json.dump({"args": vars(args), "rows": rows, "peak_tflops": peak}, open(args.json, "w"), indent=2)
    return 0


if __name__ == "__main__":
    sys.exit(main())
