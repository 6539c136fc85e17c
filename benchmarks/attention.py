"""Causal attention forward (and the library's forward + backward) on one B200.

    python benchmarks/attention.py [--batch 2] [--seq 4096] [--heads 32] [--kv-heads 4] [--dim 128] [--window 0]
        [--iters 10] [--json out.json]

Times the library path of ``ops/attention.py`` (cuDNN SDPA / flash-attn) and, when the hand-written forward is
switched on (``SLAB_ATTENTION_KERNEL=1``; ``SLAB_ATTENTION_KERNEL_BWD=1`` adds its backward), ``csrc/attention.cu`` on the
same packed-qkv inputs, checks the two outputs
against each other, and reports TFLOP/s (causal: half of the dense FLOPs; a window counts only the visible keys)
against the measured bf16 GEMM peak.  CUDA events, 3 warm-ups, median, 256 MB write between iterations (cold L2).

Reference numbers: cuDNN flash attention on B200, 64.3 ms per step in the reference's trace
(``docs/b200-vs-mi355x-ep8-gbs16-trace.html:433``); hd64 GQA backward at about 70 % of the MI355X bf16 peak
(``notes/2026-04/2026-04-21_gptoss_13_*:36-73``).
"""
from __future__ import annotations

import argparse
import json
import math
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


def visible_pairs(s: int, window: int) -> float:
    if window <= 0 or window >= s:
        return s * (s + 1) / 2.0
    return window * (window + 1) / 2.0 + (s - window) * float(window)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default="")
    a = ap.parse_args(argv)
    from system_lab_b200.ops import attention_kernel as ak, cuda as cops
    from system_lab_b200.ops.attention import _library
    dev = torch.device("cuda")
    b, s, hq, hkv, d = a.batch, a.seq, a.heads, a.kv_heads, a.dim
    qkv = torch.randn(b, s, (hq + 2 * hkv) * d, device=dev, dtype=torch.bfloat16)
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
    q, k, v = q.unflatten(-1, (hq, d)), k.unflatten(-1, (hkv, d)), v.unflatten(-1, (hkv, d))
    scale = 1.0 / math.sqrt(d)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    flops_fwd = 4.0 * b * hq * visible_pairs(s, a.window) * d
    peaks = {}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    peak = peaks.get("bf16_tflops", 1590.0)
    res = {"args": vars(a), "flops_fwd": flops_fwd, "peak_tflops": peak}

    def line(name, ms, flops):
        tf = flops / (ms * 1e9)
        res[name] = {"ms": ms, "tflops": tf, "of_peak": tf / peak}
        print(f"{name:34s} {ms:9.3f} ms {tf:9.0f} TFLOP/s  {tf / peak:5.2f} of {'measured' if peaks else 'fallback'} GEMM peak")

    line("library forward", time_cuda(lambda: _library(q, k, v, scale, a.window), flush, a.iters), flops_fwd)
    qg, kg, vg = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    g = torch.randn(b, s, hq, d, device=dev, dtype=torch.bfloat16)

    def fwd_bwd():
        qg.grad = kg.grad = vg.grad = None
        _library(qg, kg, vg, scale, a.window).backward(g)
    line("library forward + backward", time_cuda(fwd_bwd, flush, a.iters), 3.5 * flops_fwd)
    if ak._ENABLED[0] and ak.shape_ok(q, k, v, a.window) and ak.available():
        out, lse = ak.forward(q, k, v, scale, a.window)
        torch.cuda.synchronize()
        cops.check_status()
        ref = _library(q, k, v, scale, a.window)
        err = (out.float() - ref.float()).abs().max().item()
        print(f"kernel vs library: max abs difference {err:.4f}")
        res["max_abs_diff"] = err
        line("kernel forward (csrc/attention.cu)", time_cuda(lambda: ak.forward(q, k, v, scale, a.window), flush, a.iters),
             flops_fwd)
        cops.check_status()
        if ak._ENABLED_BWD[0]:
            dq, dk, dv = ak.backward(q, k, v, out, lse, g, scale, a.window)
            torch.cuda.synchronize()
            cops.check_status()
            fwd_bwd()
            errs = [(x.float() - y.float()).abs().max().item() for x, y in ((dq, qg.grad), (dk, kg.grad), (dv, vg.grad))]
            print(f"kernel vs library gradients: max abs difference dq {errs[0]:.4f} dk {errs[1]:.4f} dv {errs[2]:.4f}")
            res["grad_max_abs_diff"] = errs
            line("kernel backward (csrc/attention.cu)",
                 time_cuda(lambda: ak.backward(q, k, v, out, lse, g, scale, a.window), flush, a.iters), 2.5 * flops_fwd)
            cops.check_status()
    else:
        print("kernel forward: skipped (set SLAB_ATTENTION_KERNEL=1; needs head dim 64 / 128 and seq % 128 == 0)")
    if a.json:
        os.makedirs(os.path.dirname(a.json) or ".", exist_ok=True)
        json.dump(res, open(a.json, "w"), indent=2)
    return 0


if __name__ == "__main__":
    sys.exit(main())
