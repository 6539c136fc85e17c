"""Expert-parallel dispatch / combine microbenchmark (one process per GPU, launched by torchrun).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        benchmarks/dispatch_combine.py [--tokens 4096,8192,16384] [--hidden 7168] [--experts 256] [--topk 8]
        [--routing uniform,zipf] [--json out]

Every rank holds T tokens of `hidden` bf16 values ~N(0,1); experts are chosen by top-k over softmax of
N(0,1) router logits (`zipf` adds a Zipf(s=1.2) per-expert bias).  Timed, per op, with CUDA events on
the launching stream after warm-up, max over ranks:

* dispatch end to end: fused router kernel (top-k, counts, aux statistics) + plan (count exchange, slot
  assignment) + expert-ordered scatter + wait for every (source, expert) flag -- the whole path from router logits
  to rows in the owners' expert-major buffers;
* its parts: plan alone; scatter + wait alone, expert-ordered (bf16; per-lane stores and bulk stores) and token-ordered (bf16, and the 1x128
  block-scaled e4m3 payload with fp32 scales);
* fused combine (pull + gate-weighted top-k reduction, bf16);
* the library baseline: sort + `all_to_all_single` + receiver re-sort for dispatch, and the reverse path plus
  the weighted sum for combine (NCCL).

Roofline: bytes that must cross NVLink per rank = T * K * row_bytes * (N-1)/N, divided by (a) the peer-load
bandwidth this script measures first (every rank pulls a 256 MB shard from every peer with plain 16-byte loads,
`csrc/fsdp_comm.cu: fsdp_gather_kernel`, ingress bytes / time) and (b) the nominal 900 GB/s per direction.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

LINK_GBS_NOMINAL = 900.0


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


def measure_peer_bandwidth(mesh, world, rank, dev, sync, shard_mb: int = 256) -> float | None:
    """GB/s of NVLink ingress per rank with every rank pulling from all peers at once (plain 16-byte peer loads)."""
    if world < 2:
        return None
    from system_lab_b200.comm.fsdp_comm import FsdpPeerComm
    comm = FsdpPeerComm(mesh.ep_group, world, rank, dev)
    shard = torch.empty(shard_mb << 20, dtype=torch.uint8, device=dev).view(torch.bfloat16)
    full = torch.empty(shard.numel() * world, dtype=torch.bfloat16, device=dev)
    us = timed(lambda: comm.all_gather(full, shard), 5, 2, sync)
    # the gather also copies the local shard twice (staging + own slice): small next to (world - 1) remote shards
    return (world - 1) * shard.numel() * 2 / us / 1e3


def one_case(args, mesh, world, rank, dev, T, routing, link_gbs, sync):
    from system_lab_b200.moe.dispatch import AllToAllDispatcher
    from system_lab_b200.moe.fused_dispatch import FusedDispatcher
    from system_lab_b200.ops import cuda as cops
    H, E, K = args.hidden, args.experts, args.topk
    torch.manual_seed(1234 + rank)
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    logits = torch.randn(T, E, device=dev)
    if routing == "zipf":
        logits = logits + torch.log(1.0 / torch.arange(1, E + 1, device=dev, dtype=torch.float32) ** 1.2)
    w, idx, _, _ = cops.router_fused(logits, K, "softmax", None, True, 1.0, 1e-3)
    w, idx = w.contiguous(), idx.contiguous()
    res = {}

    def rec(name, us, bytes_cross=None):
        res[name] = {"us": us}
        line = f"  {name:44s} {us:9.1f} us"
        if bytes_cross and world > 1:
            gbs = bytes_cross / us / 1e3
            res[name].update(gbs=gbs, frac_of_nominal=gbs / LINK_GBS_NOMINAL)
            line += f"  {gbs:7.1f} GB/s/rank  {gbs / LINK_GBS_NOMINAL:5.2f} of nominal 900"
            if link_gbs:
                res[name]["frac_of_measured"] = gbs / link_gbs
                line += f"  {gbs / link_gbs:5.2f} of measured {link_gbs:.0f}"
        if rank == 0:
            print(line, flush=True)

    remote = (world - 1) / world if world > 1 else 1.0
    b_bf16 = T * K * H * 2 * remote
    b_fp8 = T * K * (H + H // 128 * 4) * remote
    fused = FusedDispatcher(mesh, E, K, H, T, 128, dev)
    plan = fused.plan(idx)

    def f_e2e():
        ww, ii, _, _ = cops.router_fused(logits, K, "softmax", None, True, 1.0, 1e-3)
        pl = fused.plan(ii)
        fused.scatter_ordered(pl, x, ww, 0).wait()
    rec("dispatch: router + plan + scatter + wait", timed(f_e2e, args.iters, args.warmup, sync), b_bf16)
    rec("  plan (count exchange + slots)", timed(lambda: fused.plan(idx), args.iters, args.warmup, sync))
    rec("  scatter + wait, expert-ordered bf16", timed(lambda: fused.scatter_ordered(plan, x, w, 0).wait(),
                                                      args.iters, args.warmup, sync), b_bf16)
    from system_lab_b200.moe.fused_dispatch import set_scatter_bulk
    set_scatter_bulk(True)
    rec("  scatter + wait, expert-ordered bf16, bulk stores", timed(lambda: fused.scatter_ordered(plan, x, w, 0).wait(),
                                                                   args.iters, args.warmup, sync), b_bf16)
    set_scatter_bulk(False)

    def f_tok():
        ep = fused.scatter(plan, x, w, 0)
        fused.wait_rows(0, ep)
    rec("  scatter + wait, token-ordered bf16", timed(f_tok, args.iters, args.warmup, sync), b_bf16)
    fused.out_rows.copy_(fused.rows[0])

    def f_comb():
        ep = fused.signal_out()
        fused.pull_rows(plan, ep, w)
    rec("combine bf16 (pull, gate-weighted)", timed(f_comb, args.iters, args.warmup, sync), b_bf16)
    torch.cuda.synchronize()
    cops.check_status()
    del fused, plan
    torch.cuda.empty_cache()
    if H % 128 == 0 and not args.no_fp8:
        fused8 = FusedDispatcher(mesh, E, K, H, T, 128, dev, fp8_payload=True)
        plan8 = fused8.plan(idx)

        def f_disp8():
            ep = fused8.scatter(plan8, x, w, 0, fp8=True)
            fused8.wait_rows(0, ep)
        rec("  scatter + wait, token-ordered fp8 1x128", timed(f_disp8, args.iters, args.warmup, sync), b_fp8)
        torch.cuda.synchronize()
        cops.check_status()
        del fused8, plan8
        torch.cuda.empty_cache()
    if not args.no_baseline:
        base = AllToAllDispatcher(mesh.ep_group if world > 1 else None, E, 128)
        pb = base.plan(idx.long())
        with torch.no_grad():
            rec("NCCL all_to_all dispatch bf16", timed(lambda: base.dispatch_rows(pb, x), args.iters, args.warmup, sync),
                b_bf16)
            xe_b = base.dispatch_rows(pb, x)
            rec("NCCL all_to_all combine bf16", timed(lambda: base.combine_rows(pb, xe_b, w), args.iters, args.warmup,
                                                      sync), b_bf16)
            rec("NCCL baseline plan (host sync)", timed(lambda: base.plan(idx.long()), args.iters, args.warmup, sync))
    counts = torch.bincount(idx.reshape(-1).long(), minlength=E).float()
    if world > 1:
        dist.all_reduce(counts)
    per_rank = counts.reshape(world, -1).sum(1)
    res["rank_load_max_over_mean"] = float(per_rank.max() / per_rank.mean())
    res["roofline_us"] = {"bf16_nominal": b_bf16 / LINK_GBS_NOMINAL / 1e3, "fp8_nominal": b_fp8 / LINK_GBS_NOMINAL / 1e3}
    if rank == 0:
        print(f"  rank load max/mean = {res['rank_load_max_over_mean']:.3f}", flush=True)
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="4096", help="comma-separated tokens per rank")
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--routing", default="uniform", help="comma-separated: uniform, zipf")
    ap.add_argument("--zipf", action="store_true", help="same as --routing zipf")
    ap.add_argument("--no-fp8", action="store_true")
    ap.add_argument("--no-baseline", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    from system_lab_b200.parallel.mesh import build_mesh, init_distributed
    rank, world, dev = init_distributed("cuda")
    mesh = build_mesh(1, world, 1)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    link = measure_peer_bandwidth(mesh, world, rank, dev, sync)
    if rank == 0 and link:
        print(f"measured peer-load bandwidth, all ranks pulling from all peers: {link:.0f} GB/s ingress per rank "
              f"(nominal {LINK_GBS_NOMINAL:.0f} per direction)", flush=True)
    routings = ["zipf"] if args.zipf else [r for r in args.routing.split(",") if r]
    out = {"world": world, "hidden": args.hidden, "experts": args.experts, "topk": args.topk,
           "peer_load_gbs_measured": link, "cases": []}
    for T in [int(t) for t in args.tokens.split(",") if t]:
        for routing in routings:
            if rank == 0:
                print(f"EP={world} T={T} H={args.hidden} E={args.experts} top-{args.topk} routing={routing}", flush=True)
            res = one_case(args, mesh, world, rank, dev, T, routing, link, sync)
            out["cases"].append({"tokens": T, "routing": routing, "results": res})
    if rank == 0 and args.json:
        os.makedirs(os.path.dirname(args.json) or ".", exist_ok=True)
        json.dump(out, open(args.json, "w"), indent=2)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
