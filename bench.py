"""Headline benchmark: MoE training tokens/s on the Qwen3-30B-A3B shaped model, one node.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun, one rank per GPU)

Metric: whole-job training tokens per second (forward + backward + AdamW step), bf16 compute,
synthetic uniform-random token ids, random-init weights, sequence length 4096, 2 sequences per GPU per
step (global batch = 2N sequences: weak scaling; N = 8 is the named global batch of 16).  The full
48-layer / 128-expert model runs at every N; what changes with N is the memory plan that lets it fit
180 GB per GPU (printed in ``config.memory_plan``).  Device time is measured with CUDA events around
exactly K steps, max over ranks.  ``e2e`` repeats the measurement through ``Trainer.train_step`` with
each step's token ids copied from pinned host memory and the step's loss read back to the host.

``--impl reference`` reports that the reference cannot run: it ships no trainer (only notes, a tuning
agent skeleton and a trace analyzer) and is not pip-installable.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

PUBLISHED_TOKENS_PER_S = 135_600.0   # reference's B200x8 trace: GPT-OSS-20B EP8, 16x8192 tokens / 0.96676 s


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--preset", default="qwen3-30b-a3b")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override layer count (invalid as a result)")
    ap.add_argument("--seqs-per-gpu", type=int, default=2)
    ap.add_argument("--pp", type=int, default=1, help="pipeline stages (DeepSeek-V3 proxy: 2)")
    ap.add_argument("--ep", type=int, default=0, help="expert parallel size (default: all data ranks)")
    ap.add_argument("--gbs", type=int, default=0, help="global batch in sequences (default: seqs-per-gpu x N)")
    ap.add_argument("--mbs", type=int, default=0, help="micro-batch in sequences (default: seqs-per-gpu)")
    ap.add_argument("--keep-dispatched", action="store_true",
                    help="when the memory estimate leaves room, keep every layer's dispatched rows (fixed-size copies of "
                         "1.5 x the balanced load) for the recomputed block; measured neutral at 2 GPUs, hence opt-in")
    ap.add_argument("--host-profile", default="",
                    help="write a cProfile summary (rank 0, by own time) of the host side of the device-timed loop to "
                         "this file; the run's numbers are then not benchmark values")
    ap.add_argument("--sync-loss-read", action="store_true",
                    help="end-to-end region: read each step's loss before launching the next step (default: the read "
                         "is collected one step later, with the next step already queued)")
    ap.add_argument("--plan", default="", help="force a memory plan by name instead of the first that fits")
    ap.add_argument("--dispatcher", default=None, help="fused | alltoall (default: preset)")
    ap.add_argument("--kernels", default="auto", help="auto | false (PyTorch/library baseline path)")
    ap.add_argument("--balanced-routing", action="store_true",
                    help="route by fixed random logits (load-balanced experts); recorded in config")
    ap.add_argument("--trace", default="", help="after timing, profile one more step into this Kineto trace")
    ap.add_argument("overrides", nargs="*")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.Q}",
                                       "--format=csv,noheader,nounits", "-lms", "200"],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self) -> dict:
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.f.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx = float(parts[2])
            except ValueError:
                continue
            for nm, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        os.unlink(self.f.name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def _min_median_max(xs):
    if not xs:
        return None
    xs = sorted(xs)
    return [round(xs[0], 2), round(xs[len(xs) // 2], 2), round(xs[-1], 2)]


def choose_memory_plan(cfg, world: int, force: str = "", allow_keep: bool = False) -> dict:
    """Highest-fidelity optimizer/weight layout that fits 92 % of 180 GB per GPU."""
    from system_lab_b200.pilot.constraints import estimate_memory
    # With one micro-batch per step the update runs inside backward in every plan: a layer's reduce-scatter is fused
    # with its AdamW step (dense groups, fp32 masters) or its AdamW runs on a side stream beside the next layer's
    # backward (expert groups), and no gradient buffer outlives its layer.  Several micro-batches (pipeline runs)
    # accumulate gradients and update after the last one.
    one_mb = cfg.train.global_batch_size == cfg.train.micro_batch_size * max(
        world // (cfg.parallel.pipeline_model_parallel_size * cfg.parallel.tensor_model_parallel_size
                  * cfg.parallel.context_parallel_size), 1)
    plans = [
        ("fp32-master+fp32-moments", dict(master_weights=True, optimizer_state_dtype="fp32"), one_mb),
        ("fp32-master+bf16-moments", dict(master_weights=True, optimizer_state_dtype="bf16"), one_mb),
        ("bf16-weights+bf16-moments", dict(master_weights=False, optimizer_state_dtype="bf16"), one_mb),
        ("bf16-weights+8bit-moments", dict(master_weights=False, optimizer_state_dtype="fp8"), one_mb),
    ]
    last = None
    # selective recompute (attention kept, feed-forward block re-run) with the best optimizer format that fits comes
    # before full recompute with a better format: re-running attention costs more than the format buys
    for gran in ("selective", "full"):
        for name, prec, in_bwd in plans:
            if force and name != force:
                continue
            for k, v in prec.items():
                setattr(cfg.precision, k, v)
            cfg.train.optimizer_in_backward = in_bwd
            cfg.precision.recompute_granularity = gran
            est = estimate_memory(cfg, world)
            # the estimate has been within a few GiB of the measured peaks; a plan must clear the 92 % line by 8 GiB
            roomy = est["fits"] and est["total_bytes"] + (8 << 30) <= 0.92 * est["hbm_bytes"]
            last = {"name": name, "optimizer_in_backward": in_bwd, "recompute": gran,
                    "est_gb": round(est["total_bytes"] / 2**30, 1), "fits": bool(roomy)}
            if roomy:
                if allow_keep and gran == "selective" and cfg.model.num_experts > 0 \
                        and cfg.model.moe_keep_dispatched_factor == 0:
                    # spare memory buys speed: keep every layer's dispatched rows so the recomputed block needs
                    # no second plan exchange and dispatch.  A fixed-size copy of 1.5 x the balanced load (one rank:
                    # the load itself); a layer whose rows do not fit on some rank is dispatched again instead.
                    ep = cfg.parallel.expert_model_parallel_size
                    cfg.model.moe_keep_dispatched_factor = 1.0 if ep <= 1 else 1.5
                    est2 = estimate_memory(cfg, world)
                    if est2["total_bytes"] + (8 << 30) <= 0.88 * est2["hbm_bytes"]:   # optional: only with headroom
                        last.update(keep_dispatched=cfg.model.moe_keep_dispatched_factor,
                                    est_gb=round(est2["total_bytes"] / 2**30, 1))
                    else:
                        cfg.model.moe_keep_dispatched_factor = 0.0
                return last
    return last


def main() -> int:
    args = parse()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "reference ships no trainer or kernels (notes + tuning-agent skeleton + trace analyzer); "
                          "pip install fails: neither setup.py nor pyproject.toml"}))
        return 0
    import torch
    import torch.distributed as dist
    from system_lab_b200.config import Config
    from system_lab_b200.parallel.mesh import build_mesh, init_distributed
    from system_lab_b200.trainer.loop import Trainer

    rank, world, dev = init_distributed("auto")
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)
    n = world
    dp = n // args.pp
    ov = [f"global_batch_size={args.gbs or args.seqs_per_gpu * n}", f"micro_batch_size={args.mbs or args.seqs_per_gpu}",
          f"expert_model_parallel_size={args.ep or dp}", f"pipeline_model_parallel_size={args.pp}", "clip_grad=1.0",
          f"use_cuda_kernels={args.kernels}"]
    if args.layers:
        ov.append(f"num_layers={args.layers}")
    if args.dispatcher:
        ov.append(f"moe_token_dispatcher_type={args.dispatcher}")
    if args.balanced_routing:
        ov.append("moe_router_force_load_balancing=true")
    cfg = Config.load(preset=args.preset, overrides=ov + list(args.overrides))
    plan = choose_memory_plan(cfg, n, args.plan, args.keep_dispatched)
    cfg.validate(n)
    mesh = build_mesh(cfg.parallel.pipeline_model_parallel_size, cfg.parallel.expert_model_parallel_size,
                      cfg.parallel.context_parallel_size, cfg.parallel.num_distributed_optimizer_instances,
                      cfg.parallel.tensor_model_parallel_size, cfg.parallel.expert_tensor_parallel_size)
    trainer = Trainer(cfg, mesh=mesh, device=dev)
    from system_lab_b200.ops import cuda as cops
    tokens_per_step = trainer.tokens_per_step

    def sync():
        if world > 1:
            dist.barrier()
        if dev.type == "cuda":
            torch.cuda.synchronize()

    # ---- warm-up --------------------------------------------------------------------------------
    for _ in range(args.warmup):
        out = trainer.train_step()
        trainer.finish_loss_read(trainer.begin_loss_read(out))     # the read path of the end-to-end region, warmed up too
        if dev.type == "cuda":
            trainer.check_device_status()      # a kernel that gave up (bounded wait, capacity) ends the run here
    # ---- device-timed region: K steps, inputs already on the device, no host read inside ----------------
    staged = []
    for i in range(args.steps):
        mbs = trainer.data.microbatches(trainer.step + i)
        staged.append([(a.to(dev), b.to(dev)) for a, b in mbs])
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))) if rank == 0 else None
    sync()
    cops_launch0 = cops.LAUNCHES[0] if hasattr(cops, "LAUNCHES") else 0
    if dev.type == "cuda":
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    last = None
    host_prof = None
    if args.host_profile and rank == 0:
        import cProfile
        host_prof = cProfile.Profile()
        host_prof.enable()
    for i in range(args.steps):
        last = trainer.train_step(batches=staged[i])
    if host_prof is not None:
        host_prof.disable()
        host_s = time.perf_counter() - t0
        import io
        import pstats
        buf = io.StringIO()
        buf.write(f"host time to launch {args.steps} steps: {host_s * 1e3 / args.steps:.1f} ms per step (under cProfile)\n")
        pstats.Stats(host_prof, stream=buf).sort_stats("tottime").print_stats(70)
        os.makedirs(os.path.dirname(args.host_profile) or ".", exist_ok=True)
        with open(args.host_profile, "w") as f:
            f.write(buf.getvalue())
    if dev.type == "cuda":
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    else:
        ms = (time.perf_counter() - t0) * 1e3
    launches = (cops.LAUNCHES[0] - cops_launch0) if hasattr(cops, "LAUNCHES") else 0
    sync()
    clocks = sampler.stop() if sampler else None
    final_loss = float(last["loss"])
    # ---- end-to-end region: pinned host inputs copied every step, loss read back every step ----------------
    sync()
    h2d = d2h = 0
    if dev.type == "cuda":
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
    t0 = time.perf_counter()
    # Every step's loss and gradient norm are read on the host, through the trainer's pinned read tickets: the copy is
    # queued behind the step, and the host collects it after it has launched the following step, so the device is not
    # left idle while the host waits (--sync-loss-read reads at once instead, as Trainer.fit does by default).
    step_ms, e2e_losses = [], []                                 # host clock between two completed reads
    pending = None
    ts = time.perf_counter()
    for i in range(args.steps):
        mbs = trainer.data.microbatches(trainer.step)          # pinned host tensors
        h2d = sum(a.numel() * a.element_size() + b.numel() * b.element_size() for a, b in mbs)
        out = trainer.train_step(batches=mbs)
        ticket = trainer.begin_loss_read(out)                    # device -> host copy of the step's result
        d2h = 3 * 4
        if args.sync_loss_read:
            e2e_losses.append(trainer.finish_loss_read(ticket)[0])
        else:
            if pending is not None:
                e2e_losses.append(trainer.finish_loss_read(pending)[0])
            pending = ticket
        if len(e2e_losses) > len(step_ms):
            now = time.perf_counter()
            step_ms.append((now - ts) * 1e3)
            ts = now
    if pending is not None:
        e2e_losses.append(trainer.finish_loss_read(pending)[0])  # the last step's numbers, inside the timed region
    if dev.type == "cuda":
        f1.record()
        torch.cuda.synchronize()
        e2e_ms = f0.elapsed_time(f1)
    else:
        e2e_ms = (time.perf_counter() - t0) * 1e3
    sync()
    if dev.type == "cuda":
        cops.check_status()
    if args.trace and rank == 0 or (args.trace and world > 1):
        acts = [torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA]
        with torch.profiler.profile(activities=acts) as prof:
            with torch.profiler.record_function("ProfilerStep#0"):
                trainer.train_step()
                torch.cuda.synchronize()
        if rank == 0:
            os.makedirs(os.path.dirname(args.trace) or ".", exist_ok=True)
            prof.export_chrome_trace(args.trace)
            with open(args.trace + ".cpu_ops.txt", "w") as f:
                f.write(prof.key_averages().table(sort_by="self_cpu_time_total", row_limit=40, max_name_column_width=60))
    load_ratio = trainer.rank_load_ratio()
    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    if rank == 0:
        ms_step = ms / args.steps
        value = tokens_per_step / (ms_step / 1e3)
        e2e_value = tokens_per_step / (e2e_ms / args.steps / 1e3)
        m = cfg.model
        line = {
            "metric": "MoE train tokens/sec/box", "value": value, "unit": "tokens/s", "n_gpus": n,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": value / PUBLISHED_TOKENS_PER_S, "dtype": "bf16",
            "data": "synthetic uniform-random token ids, random-init N(0,0.02) weights",
            "impl": "ours",
            "config": {"model": m.name, "num_layers": m.num_layers, "hidden": m.hidden_size,
                       "num_experts": m.num_experts, "topk": m.moe_router_topk, "global_batch": cfg.train.global_batch_size,
                       "seq_len": m.seq_length, "parallelism": f"fsdp+ep{mesh.ep}" + (f"+pp{mesh.pp}" if mesh.pp > 1 else "") + (f"+tp{mesh.tp}" if mesh.tp > 1 else ""),
                       "memory_plan": plan, "recompute": cfg.precision.recompute_granularity,
                       "dispatcher": m.moe_token_dispatcher_type, "kernels": args.kernels,
                       "routing": "forced-balanced" if m.moe_router_force_load_balancing else "learned-router",
                       "ep_rank_load_max_over_mean": load_ratio,
                       "l2": "working set (weights + activations) is far larger than the 126 MB L2",
                       "tflops_per_gpu": value / n * trainer.flops_per_token / 1e12,
                       "final_loss": final_loss,
                       "baseline_note": "vs_baseline divides by the reference's only B200 number: GPT-OSS-20B "
                                        "EP8 step of 966.76 ms = 135.6k tokens/s/box (a different model)"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / args.steps,
                    "loss_read": "at once" if args.sync_loss_read else "pinned buffer, collected after the next step's launch",
                    "losses_read": len(e2e_losses), "last_loss": e2e_losses[-1] if e2e_losses else None,
                    # host time between two collected reads; the first interval also holds the launch of the second
                    # step (reads are collected one step behind) and is left out
                    "rank0_step_ms_min_median_max": _min_median_max(step_ms[1:] if len(step_ms) > 2 else step_ms)},
            "gpu_launches": launches,
            "mem_peak_gb": torch.cuda.max_memory_allocated() / 2**30 if dev.type == "cuda" else 0.0,
            "expert_relocations": trainer.relocator.history if trainer.relocator else [],
            "kept_dispatch_fallbacks": getattr(trainer.engine.dispatcher, "keep_fallbacks", 0),
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
