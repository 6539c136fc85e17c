"""Expert-parallel dispatch / combine microbenchmark (one process per GPU, launched by torchrun).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        benchmarks/dispatch_combine.py [--tokens 4096] [--hidden 7168] [--experts 256] [--topk 8] [--zipf] [--json out]

Every rank holds T tokens of `hidden` bf16 values ~N(0,1); experts are chosen by top-k over softmax of
N(0,1) router logits (`--zipf` adds a Zipf(s=1.2) per-expert bias).  Timed, per op, with CUDA events on
the launching stream after warm-up, max over ranks:

* fused dispatch, bf16 payload and 1x128 block-scaled e4m3 payload (+ fp32 scales), including the wait for
  every source's rows;
* fused combine (pull + gate-weighted top-k reduction, bf16);
* the plan (count exchange + slot assignment);
* the library baseline: sort + `all_to_all_single` + receiver re-sort for dispatch, and the reverse path plus
  the weighted sum for combine (NCCL).

Roofline: bytes that must cross NVLink per rank = T * K * row_bytes * (N-1)/N at the measured 770 GB/s per
direction (900 nominal).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

LINK_GBS_MEASURED = 770.0


def timed(fn, iters, warmup, sync):
    for _ in range(warmup):
        fn()
    sync()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--zipf", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    from system_lab_b200.moe.dispatch import AllToAllDispatcher
    from system_lab_b200.moe.fused_dispatch import FusedDispatcher
    from system_lab_b200.ops import cuda as cops
    from system_lab_b200.parallel.mesh import build_mesh, init_distributed
    rank, world, dev = init_distributed("cuda")
    mesh = build_mesh(1, world, 1)
    T, H, E, K = args.tokens, args.hidden, args.experts, args.topk
    torch.manual_seed(1234 + rank)
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    logits = torch.randn(T, E, device=dev)
    if args.zipf:
        logits = logits + torch.log(1.0 / torch.arange(1, E + 1, device=dev, dtype=torch.float32) ** 1.2)
    probs = torch.softmax(logits, -1)
    w, idx = torch.topk(probs, K, dim=-1)
    w = (w / w.sum(-1, keepdim=True)).contiguous()
    idx = idx.int().contiguous()

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    fused = FusedDispatcher(mesh, E, K, H, T, 128, dev)
    fused8 = FusedDispatcher(mesh, E, K, H, T, 128, dev, fp8_payload=True) if H % 128 == 0 else None
    base = AllToAllDispatcher(mesh.ep_group if world > 1 else None, E, 128)
    plan = fused.plan(idx)
    plan8 = fused8.plan(idx) if fused8 else None
    pb = base.plan(idx.long())
    res = {}

    def rec(name, us, bytes_cross=None):
        res[name] = {"us": us}
        line = f"{name:34s} {us:9.1f} us"
        if bytes_cross:
            gbs = bytes_cross / us / 1e3
            res[name].update(gbs=gbs, frac_of_link=gbs / LINK_GBS_MEASURED)
            line += f"  {gbs:7.1f} GB/s per rank  {gbs / LINK_GBS_MEASURED:5.2f} of measured NVLink (770 GB/s/dir)"
        if rank == 0:
            print(line, flush=True)

    remote = (world - 1) / world if world > 1 else 1.0
    b_bf16 = T * K * H * 2 * remote
    b_fp8 = T * K * (H + H // 128 * 4) * remote

    def f_plan():
        fused.plan(idx)
    rec("fused plan (counts+slots)", timed(f_plan, args.iters, args.warmup, sync))

    def f_disp():
        ep = fused.scatter(plan, x, w, 0)
        fused.wait_rows(0, ep)
    rec("fused dispatch bf16", timed(f_disp, args.iters, args.warmup, sync), b_bf16)
    if fused8:
        def f_disp8():
            ep = fused8.scatter(plan8, x, w, 0, fp8=True)
            fused8.wait_rows(0, ep)
        rec("fused dispatch fp8 1x128", timed(f_disp8, args.iters, args.warmup, sync), b_fp8)
    fused.out_rows.copy_(fused.rows[0])

    def f_comb():
        ep = fused.signal_out()
        fused.pull_rows(plan, ep, w)
    rec("fused combine bf16 (weighted)", timed(f_comb, args.iters, args.warmup, sync), b_bf16)

    with torch.no_grad():
        def b_disp():
            return base.dispatch_rows(pb, x)
        rec("NCCL all_to_all dispatch bf16", timed(b_disp, args.iters, args.warmup, sync), b_bf16)
        xe_b = base.dispatch_rows(pb, x)

        def b_comb():
            base.combine_rows(pb, xe_b, w)
        rec("NCCL all_to_all combine bf16", timed(b_comb, args.iters, args.warmup, sync), b_bf16)

        def b_plan():
            base.plan(idx.long())
        rec("NCCL baseline plan (host sync)", timed(b_plan, args.iters, args.warmup, sync))
    torch.cuda.synchronize()
    cops.check_status()
    # load statistics of this routing
    counts = torch.bincount(idx.reshape(-1).long(), minlength=E).float()
    if world > 1:
        dist.all_reduce(counts)
    per_rank = counts.reshape(world, -1).sum(1)
    res["rank_load_max_over_mean"] = float(per_rank.max() / per_rank.mean())
    if rank == 0:
        print(f"rank load max/mean = {res['rank_load_max_over_mean']:.3f}; roofline dispatch bf16 "
              f"{b_bf16 / LINK_GBS_MEASURED / 1e3:.0f} us, fp8 {b_fp8 / LINK_GBS_MEASURED / 1e3:.0f} us", flush=True)
        if args.json:
            os.makedirs(os.path.dirname(args.json) or ".", exist_ok=True)
            json.dump({"args": vars(args), "world": world, "results": res}, open(args.json, "w"), indent=2)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
