"""One MoE layer end to end: router -> dispatch -> expert fc1 -> SwiGLU x gate -> expert fc2 -> combine, forward and
forward + backward, on N expert-parallel ranks (one process per GPU under torchrun; one process without it).

    python benchmarks/moe_layer.py [--tokens 4096] [--hidden 7168] [--ffn 2048] [--experts 256] [--topk 8]
        [--dispatcher fused|alltoall] [--no-push] [--balanced] [--iters 10] [--json out.json] [--device cuda|cpu]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        benchmarks/moe_layer.py --tokens 4096

Timed with CUDA events on the launching stream (3 warm-ups, median, max over ranks; a 256 MB write between
iterations keeps L2 cold).  Reported per pass: milliseconds, expert-GEMM TFLOP/s per GPU counted on the rows the rank
actually received, and the share of the time a perfectly overlapped layer would need (the slower of the GEMM time
at the measured bf16 rate and the NVLink time of the dispatch + combine bytes at 770 GB/s per direction).
On CPU (``--device cpu``) the same script runs the library path on tiny shapes: a logic check, not a measurement.

Reference counterparts: the end-to-end MoE micro-benchmarks ``test_moe_e2e*.hip`` and the 8-GPU baseline
``bench_moe_baseline_8gpu.py`` (``notes/2026-04/2026-04-14_moe_e2e_performance_benchmark.md:15-19,95``;
per-rank payload table ``notes/2026-04/2026-04-14_moe_comm_overlap_analysis.md:28-33``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

LINK_GBS_MEASURED = 770.0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096, help="tokens per rank")
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--ffn", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--dispatcher", default="fused", choices=["fused", "alltoall"])
    ap.add_argument("--no-push", action="store_true", help="pull combine instead of the GEMM's push epilogue")
    ap.add_argument("--balanced", action="store_true", help="route by a fixed random table (balanced load)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--json", default="")
    args = ap.parse_args(argv)

    from system_lab_b200.config import Config
    from system_lab_b200.parallel.mesh import init_distributed
    from system_lab_b200.trainer.loop import Trainer
    rank, world, dev = init_distributed(args.device)
    cuda = dev.type == "cuda"
    seq = 128 if args.tokens % 128 == 0 else args.tokens
    ov = ["num_layers=1", f"hidden_size={args.hidden}", f"moe_ffn_hidden_size={args.ffn}", f"num_experts={args.experts}",
          f"moe_router_topk={args.topk}", f"seq_length={seq}", f"micro_batch_size={args.tokens // seq}",
          f"global_batch_size={args.tokens // seq * world}", f"expert_model_parallel_size={world}",
          f"params_dtype={'bf16' if cuda else 'fp32'}", f"moe_token_dispatcher_type={args.dispatcher if cuda else 'alltoall'}",
          f"moe_combine_push={'false' if args.no_push else 'true'}", f"moe_pad_expert_rows_to={128 if cuda else 1}",
          f"moe_router_force_load_balancing={'true' if args.balanced else 'false'}", "recompute_granularity=none",
          "vocab_size=1024", "num_attention_heads=2", "num_query_groups=2", "kv_channels=64", f"device={args.device}",
          "first_k_dense=0", "moe_shared_expert_intermediate_size=0"]
    cfg = Config.load(preset="simplemoe-tiny", overrides=ov)
    tr = Trainer(cfg)
    layer = tr.engine.layer_units[0]
    layer.gather()
    ffn = tr.engine.moe_ffns()[0]
    dtype = torch.bfloat16 if cuda else torch.float32
    torch.manual_seed(1234 + rank)
    x = torch.randn(args.tokens, args.hidden, device=dev, dtype=dtype, requires_grad=True)
    g = torch.randn(args.tokens, args.hidden, device=dev, dtype=dtype)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev) if cuda else None

    def sync():
        if cuda:
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def fwd():
        with torch.no_grad():
            return ffn(x)

    def fwd_bwd():
        layer.prepare_grads()
        x.grad = None
        ffn(x).backward(g)

    def timed(fn):
        for _ in range(3):
            fn()
        sync()
        ts = []
        for _ in range(args.iters):
            if cuda:
                flush.zero_()
                sync()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            else:
                sync()
                t0 = time.perf_counter()
                fn()
                ts.append((time.perf_counter() - t0) * 1e3)
        ts.sort()
        t = torch.tensor([ts[len(ts) // 2]], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    t_f = timed(fwd)
    t_fb = timed(fwd_bwd)
    if cuda:
        from system_lab_b200.ops import cuda as cops
        cops.check_status()
    # rows every rank's experts received in the last pass: each rank knows the pairs it routed to every expert
    tpe = ffn.last_tokens_per_expert.float().clone()
    if world > 1:
        dist.all_reduce(tpe)
    rows_max = float(tpe.view(world, args.experts // world).sum(1).max())
    flops_fwd = 2.0 * rows_max * 3 * args.hidden * args.ffn
    peaks = {}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    peak_tf = peaks.get("bf16_tflops", 1590.0)
    link_bytes = args.tokens * args.topk * args.hidden * 2 * (world - 1) / max(world, 1)
    t_link = link_bytes / (LINK_GBS_MEASURED * 1e6)                    # one direction, one exchange, ms
    floor_f = max(flops_fwd / (peak_tf * 1e9), 2 * t_link if world > 1 else 0.0)
    floor_fb = max(3 * flops_fwd / (peak_tf * 1e9), 4 * t_link if world > 1 else 0.0)
    res = {"world": world, "tokens_per_rank": args.tokens, "hidden": args.hidden, "ffn": args.ffn,
           "experts": args.experts, "topk": args.topk, "dispatcher": cfg.model.moe_token_dispatcher_type,
           "push": bool(cfg.model.moe_combine_push and world > 1 and cfg.model.moe_token_dispatcher_type == "fused"),
           "rows_most_loaded_rank": rows_max,
           "rows_balanced": args.tokens * args.topk,
           "fwd_ms": t_f, "fwd_bwd_ms": t_fb,
           "fwd_expert_tflops": flops_fwd / (t_f * 1e9), "fwd_bwd_expert_tflops": 3 * flops_fwd / (t_fb * 1e9),
           "fwd_floor_ms": floor_f, "fwd_bwd_floor_ms": floor_fb,
           "fwd_of_floor": floor_f / t_f, "fwd_bwd_of_floor": floor_fb / t_fb,
           "peak_source": "measured" if peaks else "fallback"}
    if rank == 0:
        print(f"MoE layer, {world} rank(s), {args.tokens} tokens/rank, hidden {args.hidden}, ffn {args.ffn}, "
              f"{args.experts} experts top-{args.topk}, dispatcher {res['dispatcher']}" + (" + push" if res["push"] else ""))
        print(f"  rows on the most loaded rank: {rows_max:.0f} (balanced: {res['rows_balanced']})")
        print(f"  forward            {t_f:9.3f} ms   {res['fwd_expert_tflops']:8.1f} TFLOP/s expert GEMMs   "
              f"{res['fwd_of_floor']:.2f} of the overlapped floor ({floor_f:.3f} ms, {res['peak_source']} peaks)")
        print(f"  forward + backward {t_fb:9.3f} ms   {res['fwd_bwd_expert_tflops']:8.1f} TFLOP/s expert GEMMs   "
              f"{res['fwd_bwd_of_floor']:.2f} of the overlapped floor ({floor_fb:.3f} ms)")
        if args.json:
            os.makedirs(os.path.dirname(args.json) or ".", exist_ok=True)
            json.dump(res, open(args.json, "w"), indent=2)
    tr.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
