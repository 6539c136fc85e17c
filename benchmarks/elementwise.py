"""Roofline of the bandwidth-bound kernels: RMSNorm (+residual), SwiGLU x probs, RoPE, quantisers, sum of squares
and the fused AdamW, each against the measured copy bandwidth.

    python benchmarks/elementwise.py [--rows 16384] [--hidden 7168] [--ffn 2048] [--params 268435456] [--json out.json]

Timing: CUDA events on the launching stream, 3 warm-ups, median of 10, a 256 MB write between iterations so the
126 MB L2 is cold.  "bytes" is the algorithmic traffic (every operand read once, every result written once);
achieved = bytes / time; the denominator is ``hbm_gbs`` of MEASURED_PEAKS.json (6650 GB/s if the file is absent).
Reference counterparts and their measured numbers: RMSNorm ``notes/2026-04/2026-04-20_gptoss_02_triton_rmsnorm_
optimization.md:54-60``, fused residual+RMSNorm ``...gptoss_18...``, SwiGLU no-cat ``...gptoss_23...:41``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def time_cuda(fn, flush, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
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
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--ffn", type=int, default=2048)
    ap.add_argument("--params", type=int, default=256 * 1024 * 1024, help="elements of the flat AdamW shard")
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    from system_lab_b200.ops import cuda as cops
    from system_lab_b200.trainer.optim import _Moment
    dev = torch.device("cuda")
    peaks = {}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    peak = peaks.get("hbm_gbs", 6650.0)
    src = "measured" if peaks else "fallback"
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    r, h, f = args.rows, args.hidden, args.ffn
    bf = torch.bfloat16
    results = {}

    def rec(name, ms, nbytes):
        gbs = nbytes / ms / 1e6
        results[name] = {"ms": ms, "bytes": nbytes, "gbs": gbs, "frac_of_copy": gbs / peak}
        print(f"{name:34s} {ms * 1e3:9.1f} us  {nbytes / 1e6:9.1f} MB  {gbs:8.0f} GB/s  {gbs / peak:5.2f} of {src} copy")

    x = torch.randn(r, h, device=dev, dtype=bf)
    res = torch.randn(r, h, device=dev, dtype=bf)
    w = torch.ones(h, device=dev, dtype=bf)
    dy = torch.randn(r, h, device=dev, dtype=bf)
    # ---- RMSNorm ----------------------------------------------------------------------------------------------------
    rec("rmsnorm fwd", time_cuda(lambda: cops.rmsnorm(x, w, 1e-6), flush), 2 * r * h * 2)
    xg = x.clone().requires_grad_(True)
    wg = w.clone().requires_grad_(True)
    y = cops.rmsnorm(xg, wg, 1e-6)
    rec("rmsnorm bwd (dx + dgamma)", time_cuda(lambda: torch.autograd.grad(y, (xg, wg), dy, retain_graph=True), flush),
        3 * r * h * 2)
    rec("residual + rmsnorm fwd", time_cuda(lambda: cops.rmsnorm_residual(x, res, w, 1e-6), flush), 4 * r * h * 2)
    # ---- SwiGLU x probs -----------------------------------------------------------------------------------------------
    gu = torch.randn(r, 2 * f, device=dev, dtype=bf)
    p = torch.rand(r, device=dev)
    rec("swiglu*probs fwd", time_cuda(lambda: cops.swiglu_probs(gu, p), flush), r * (2 * f + f) * 2 + r * 4)
    gug = gu.clone().requires_grad_(True)
    pg = p.clone().requires_grad_(True)
    out = cops.swiglu_probs(gug, pg)
    dout = torch.randn(r, f, device=dev, dtype=bf)
    rec("swiglu*probs bwd (no cat)", time_cuda(lambda: torch.autograd.grad(out, (gug, pg), dout, retain_graph=True), flush),
        r * (f + 2 * f + 2 * f) * 2 + 2 * r * 4)
    # ---- quantisers -----------------------------------------------------------------------------------------------------
    rec("quant_rowwise [rows, hidden]", time_cuda(lambda: cops.quant_rowwise(x), flush), r * h * 3 + r * 4)
    rec("quant_1x128 [rows, hidden]", time_cuda(lambda: cops.quant_1x128(x), flush), r * h * 3 + r * (h // 128) * 4)
    # ---- sum of squares ----------------------------------------------------------------------------------------------------
    n = args.params
    g32 = torch.randn(n, device=dev) * 1e-2
    acc = torch.zeros(1, device=dev)
    rec("sumsq fp32", time_cuda(lambda: cops.sumsq(g32, 1.0, acc), flush), n * 4)
    # ---- fused AdamW -----------------------------------------------------------------------------------------------------

    class G:
        pass
    for kind, pdt, gdt, name in (("fp32", torch.float32, torch.bfloat16, "adamw fp32 master+moments, bf16 grad, bf16 copy out"),
                                 ("bf16", bf, bf, "adamw bf16 weights, bf16 moments"),
                                 ("fp8", bf, bf, "adamw bf16 weights, 8-bit moments")):
        grp = G()
        grp.shard = (0.02 * torch.randn(n, device=dev)).to(pdt)
        grp.sharded = True
        grp.full = grp.shard
        grp.shard_lp = torch.empty(n, device=dev, dtype=bf) if pdt == torch.float32 else None
        grp.grad_shard = (1e-2 * torch.randn(n, device=dev)).to(gdt)
        m, v = _Moment(n, kind, dev), _Moment(n, kind, dev, sqrt_domain=(kind != "fp32"))
        coef = torch.tensor(1.0, device=dev)
        pb = 4 if pdt == torch.float32 else 2
        mb = {"fp32": 4, "bf16": 2, "fp8": 1}[kind]
        nbytes = n * (2 * pb + 2 + 4 * mb + (2 if pdt == torch.float32 else 0)) + (n // 128 * 16 if kind == "fp8" else 0)
        step = [0]

        def run(grp=grp, m=m, v=v, coef=coef):
            step[0] += 1
            cops.adamw_flat(grp, m, v, coef, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step[0])
        rec(name, time_cuda(run, flush), nbytes)
        del grp, m, v
        torch.cuda.empty_cache()
    cops.check_status()
    if args.json:
        os.makedirs(os.path.dirname(args.json) or ".", exist_ok=True)
        json.dump({"args": vars(args), "results": results, "copy_gbs": peak, "copy_source": src}, open(args.json, "w"), indent=2)


if __name__ == "__main__":
    main()
