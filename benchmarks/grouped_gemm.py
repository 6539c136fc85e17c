"""Dropless grouped expert GEMM benchmark (one B200).

32 local experts, hidden 7168 -> gate+up 4096 -> (SwiGLU) -> 2048 -> hidden 7168; per-expert token counts
drawn from a multinomial over 16384 routed slots with uniform or Zipf(s=1.2) probabilities.  Times the
forward, dgrad and wgrad kernels of both linears with CUDA events (L2 flushed between iterations) and
reports TFLOP/s against the measured cuBLAS bf16 peak; ``--baseline`` also times the library path
(``torch._grouped_mm`` if present, else a per-expert loop of ``torch.matmul``).

    python benchmarks/grouped_gemm.py [--slots 16384] [--experts 32] [--hidden 7168] [--ffn 2048] [--zipf] [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def make_counts(slots: int, experts: int, zipf: bool, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    if zipf:
        p = 1.0 / torch.arange(1, experts + 1, dtype=torch.float64) ** 1.2
    else:
        p = torch.ones(experts, dtype=torch.float64)
    idx = torch.multinomial(p / p.sum(), slots, replacement=True, generator=g)
    return torch.bincount(idx, minlength=experts).int()


ONLY = [""]
WARMUP = [3]


def time_cuda(fn, iters: int = 10, warmup: int = 3, flush=None, name: str = ""):
    if ONLY[0] and name != ONLY[0]:
        return None
    warmup = WARMUP[0]
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--slots", type=int, default=16384)
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--ffn", type=int, default=2048)
    ap.add_argument("--zipf", action="store_true")
    ap.add_argument("--baseline", action="store_true")
    ap.add_argument("--fp8", action="store_true", help="also time the block-scaled fp8 forward kernels")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default="")
    ap.add_argument("--only", default="", help="run a single op, e.g. 'fc1 fwd' (for profiler captures)")
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    ONLY[0] = args.only
    WARMUP[0] = args.warmup
    from system_lab_b200.ops import cuda as cops
    dev = torch.device("cuda")
    peaks = {}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    peak_tf = peaks.get("bf16_tflops", 1590.0)
    peak_src = "measured" if peaks else "fallback"
    counts = make_counts(args.slots, args.experts, args.zipf)
    padded = (counts + 127) // 128 * 128
    offsets = (torch.cumsum(padded, 0) - padded).int()
    rows = int(padded.sum())
    e, h, f = args.experts, args.hidden, args.ffn
    x = torch.zeros(rows, h, device=dev, dtype=torch.bfloat16)
    for o, c in zip(offsets.tolist(), counts.tolist()):
        x[o:o + c].normal_()
    w1 = (0.02 * torch.randn(e, 2 * f, h, device=dev)).to(torch.bfloat16)
    w2 = (0.02 * torch.randn(e, h, f, device=dev)).to(torch.bfloat16)
    off_d, cnt_d = offsets.to(dev), counts.to(dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    h1 = cops.grouped_gemm_raw(0, x, w1, off_d, cnt_d, 2 * f, h)
    act = torch.zeros(rows, f, device=dev, dtype=torch.bfloat16)
    act.copy_(h1[:, :f])
    dy2 = torch.zeros(rows, h, device=dev, dtype=torch.bfloat16)
    dy2.copy_(x)
    dy1 = h1.clone()
    valid = int(counts.sum())
    results = {}

    def rec(name, ms, flops):
        if ms is None:
            return
        tf = flops / ms / 1e9
        results[name] = {"ms": ms, "tflops": tf, "frac_of_peak": tf / peak_tf}
        print(f"{name:28s} {ms:8.3f} ms  {tf:8.1f} TFLOP/s  {tf / peak_tf:5.2f} of {peak_src} bf16 peak")

    fl1 = 2.0 * valid * (2 * f) * h
    fl2 = 2.0 * valid * h * f
    rec("fc1_fwd", time_cuda(lambda: cops.grouped_gemm_raw(0, x, w1, off_d, cnt_d, 2 * f, h), args.iters, flush=flush, name="fc1_fwd"), fl1)
    rec("fc2_fwd", time_cuda(lambda: cops.grouped_gemm_raw(0, act, w2, off_d, cnt_d, h, f), args.iters, flush=flush, name="fc2_fwd"), fl2)
    rec("fc1_dgrad", time_cuda(lambda: cops.grouped_gemm_raw(1, dy1, w1, off_d, cnt_d, 2 * f, h), args.iters, flush=flush, name="fc1_dgrad"), fl1)
    rec("fc2_dgrad", time_cuda(lambda: cops.grouped_gemm_raw(1, dy2, w2, off_d, cnt_d, h, f), args.iters, flush=flush, name="fc2_dgrad"), fl2)
    rec("fc1_wgrad", time_cuda(lambda: cops.grouped_gemm_raw(2, dy1, x, off_d, cnt_d, 2 * f, h), args.iters, flush=flush, name="fc1_wgrad"), fl1)
    rec("fc2_wgrad", time_cuda(lambda: cops.grouped_gemm_raw(2, dy2, act, off_d, cnt_d, h, f), args.iters, flush=flush, name="fc2_wgrad"), fl2)
    if not args.only:
        fwd_ms = results["fc1_fwd"]["ms"] + results["fc2_fwd"]["ms"]
        all_ms = sum(r["ms"] for r in results.values())
        rec("forward (fc1+fc2)", fwd_ms, fl1 + fl2)
        rec("forward+backward", all_ms, 3 * (fl1 + fl2))
    cops.check_status()
    if args.fp8:
        xq, xs = cops.quant_1x128(x)
        aq, as_ = cops.quant_1x128(act)
        w1q, w1s = cops.quant_128x128(w1)
        w2q, w2s = cops.quant_128x128(w2)
        rec("fc1_fwd_fp8", time_cuda(lambda: cops.grouped_gemm_fp8_raw(xq, xs, w1q, w1s, off_d, cnt_d), args.iters,
                                     flush=flush, name="fc1_fwd_fp8"), fl1)
        rec("fc2_fwd_fp8", time_cuda(lambda: cops.grouped_gemm_fp8_raw(aq, as_, w2q, w2s, off_d, cnt_d), args.iters,
                                     flush=flush, name="fc2_fwd_fp8"), fl2)
        xr, xrs = cops.quant_rowwise(x)
        ar, ars = cops.quant_rowwise(act)
        w1r, w1rs = cops.quant_rowwise(w1)
        w2r, w2rs = cops.quant_rowwise(w2)
        rec("fc1_fwd_fp8_rowwise", time_cuda(lambda: cops.grouped_gemm_fp8_rowwise_raw(xr, xrs, w1r, w1rs, off_d, cnt_d),
                                             args.iters, flush=flush, name="fc1_fwd_fp8_rowwise"), fl1)
        rec("fc2_fwd_fp8_rowwise", time_cuda(lambda: cops.grouped_gemm_fp8_rowwise_raw(ar, ars, w2r, w2rs, off_d, cnt_d),
                                             args.iters, flush=flush, name="fc2_fwd_fp8_rowwise"), fl2)
        # input gradients on the fp8 path: dY quantised per row, the weight from its cached [E, K, N] e4m3 copy
        g1q, g1s = cops.quant_rowwise(dy1)
        g2q, g2s = cops.quant_rowwise(dy2)
        w1t, w1ts = cops._transposed_rowwise_weight(w1)
        w2t, w2ts = cops._transposed_rowwise_weight(w2)
        rec("fc1_dgrad_fp8_rowwise", time_cuda(lambda: cops.grouped_gemm_fp8_rowwise_raw(g1q, g1s, w1t, w1ts, off_d, cnt_d),
                                               args.iters, flush=flush, name="fc1_dgrad_fp8_rowwise"), fl1)
        rec("fc2_dgrad_fp8_rowwise", time_cuda(lambda: cops.grouped_gemm_fp8_rowwise_raw(g2q, g2s, w2t, w2ts, off_d, cnt_d),
                                               args.iters, flush=flush, name="fc2_dgrad_fp8_rowwise"), fl2)
        rec("quant_rowwise dY1", time_cuda(lambda: cops.quant_rowwise(dy1), args.iters, flush=flush, name="quant_row_dy1"), 0.0)
        rec("quant_rowwise x", time_cuda(lambda: cops.quant_rowwise(x), args.iters, flush=flush, name="quant_row_x"), 0.0)
        rec("quant_1x128 x", time_cuda(lambda: cops.quant_1x128(x), args.iters, flush=flush, name="quant_x"), 0.0)
        rec("quant_128x128 w1", time_cuda(lambda: cops.quant_128x128(w1), args.iters, flush=flush, name="quant_w1"), 0.0)
        cops.check_status()
    if args.baseline and not args.only:
        cl = counts.tolist()
        ol = offsets.tolist()

        def loop_fwd(a, w):
            for i, (o, c) in enumerate(zip(ol, cl)):
                if c:
                    torch.matmul(a[o:o + c], w[i].t())
        rec("library fc1 fwd (loop)", time_cuda(lambda: loop_fwd(x, w1), args.iters, flush=flush), fl1)
        rec("library fc2 fwd (loop)", time_cuda(lambda: loop_fwd(act, w2), args.iters, flush=flush), fl2)
        big_a = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)
        big_b = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)
        rec("cuBLAS 8192^3", time_cuda(lambda: torch.matmul(big_a, big_b), args.iters), 2.0 * 8192 ** 3)
    if args.json:
        os.makedirs(os.path.dirname(args.json) or ".", exist_ok=True)
        json.dump({"args": vars(args), "results": results, "peak_tflops": peak_tf, "peak_source": peak_src},
                  open(args.json, "w"), indent=2)


if __name__ == "__main__":
    main()
