"""Snapshot export: the metric contract between a training run and the tuner.

Field names and required/conditional rules follow ``skills/pilot/workflow/observe.md:36-163``:
required fields are always present (``None`` where unobtainable), the first 20 steps are warm-up
and excluded from averages, the loss curve is down-sampled to one point per 10 steps,
``confidence_in_metrics`` is ``low`` under 50 completed steps.
"""
from __future__ import annotations

import os
import time

import torch

WARMUP_STEPS = 20
LOSS_EVERY = 10
_ENV_PREFIXES = ("NCCL_", "TORCH_NCCL_", "CUDA_", "PYTORCH_CUDA_", "OMP_", "SLAB_")


def ema(values, alpha: float = 0.1):
    out = None
    for v in values:
        out = v if out is None else alpha * v + (1 - alpha) * out
    return out


def build_snapshot(trainer, *, job_id: str = "", plan_id: str = "", session_id: str = "", round_id: int = 0,
                   mode: str = "baseline", status: str = "ok", exit_code: int = 0,
                   early_stop_reason=None, comm: dict | None = None) -> dict:
    times = trainer.step_times_ms
    steady = times[WARMUP_STEPS:] if len(times) > WARMUP_STEPS else times[len(times) // 2:]
    step_ms = sum(steady) / len(steady) if steady else None
    tok = trainer.tokens_per_step
    tps_series = [tok / (t / 1e3) for t in steady]
    cuda = trainer.device.type == "cuda"
    gib = 2**30
    mem_peak = torch.cuda.max_memory_allocated() / gib if cuda else 0.0
    mem_alloc = torch.cuda.memory_allocated() / gib if cuda else 0.0
    mem_res = torch.cuda.memory_reserved() / gib if cuda else 0.0
    curve = [[i + 1, l] for i, l in enumerate(trainer.loss_curve) if (i + 1) % LOSS_EVERY == 0 or i == 0
             or i + 1 == len(trainer.loss_curve)]
    losses = trainer.loss_curve
    has_nan = any(l != l for l in losses)
    has_inf = any(abs(l) == float("inf") for l in losses)
    moe = trainer.cfg.model.num_experts > 0
    imb = None
    if moe and trainer._tpe_accum is not None:
        tpe = trainer._tpe_accum.float()
        per_layer = tpe.max(dim=1).values / tpe.min(dim=1).values.clamp_min(1.0) - 1.0
        imb = float(per_layer.mean() * 100.0)
    expected = None
    if cuda:
        # analytic expectation for this config on B200 (achieved kernel rates, measured rank load): DIAGNOSE's
        # "tps < 0.8 x expected" soft signal compares against it
        from ..pilot.perf_model import expected_tps
        ratio = (trainer.rank_load_ratio() or 1.0) if (moe and trainer.mesh.ep > 1) else 1.0
        try:
            expected = expected_tps(trainer.cfg, trainer.mesh.world, rank_load_ratio=ratio)
        except (ZeroDivisionError, KeyError, ValueError):
            expected = None
    comm = comm or {}
    completed = len(times)
    return {
        "job_id": job_id, "plan_id": plan_id, "session_id": session_id, "round": round_id, "mode": mode,
        "finished_at": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()),
        "status": status, "exit_code": exit_code, "early_stop_reason": early_stop_reason,
        "completed_steps": completed, "wall_time_s": sum(times) / 1e3,
        "confidence_in_metrics": "low" if completed < 50 else ("medium" if completed < 200 else "high"),
        "metrics": {
            "tps": (tok / (step_ms / 1e3)) if step_ms else None,
            "step_time_ms": step_ms,
            "expected_tps": expected,
            "tps_ema_50": ema(tps_series[-50:]) if tps_series else None,
            "tps_ema_full": ema(tps_series) if tps_series else None,
            "tflops_per_gpu": (tok / (step_ms / 1e3) / trainer.mesh.world * trainer.flops_per_token / 1e12)
            if step_ms else None,
            "gpu_util_avg": comm.get("gpu_util_avg"),
            "intra_node_util_avg": comm.get("intra_node_util_avg"),
            "inter_node_util_avg": None,
            "cpu_wait_time_pct": comm.get("cpu_wait_time_pct"),
            "kernel_launch_overhead_pct": comm.get("kernel_launch_overhead_pct"),
            "mem_peak_gb": mem_peak, "mem_alloc_avg_gb": mem_alloc, "mem_reserved_avg_gb": mem_res,
            "mem_reserved_to_alloc_ratio": (mem_res / mem_alloc) if mem_alloc > 0 else None,
            "has_oom_event": False,
            "comm_ratio": comm.get("comm_ratio"),
            "bubble_ratio": comm.get("bubble_ratio", 0.0 if trainer.mesh.pp == 1 else None),
            "overlap_ratio": comm.get("overlap_ratio"),
            "ar_share_pct": comm.get("ar_share_pct"),
            "alltoall_share_pct": comm.get("alltoall_share_pct"),
            "has_nan": has_nan, "has_inf": has_inf,
            "expert_load_imbalance_pct": imb,
            "expert_drop_rate_pct": 0.0 if moe else None,      # dropless by construction
            "alltoall_skew_pct": None,
        },
        "loss": {"curve": curve, "ema_50": ema(losses[-50:]) if losses else None,
                 "ema_full": ema(losses) if losses else None, "drift_vs_reference": None},
        "resolved_env": {k: v for k, v in sorted(os.environ.items()) if k.startswith(_ENV_PREFIXES)},
        "resolved_config": trainer.cfg.to_dict(),
        "artifacts": {"stdout": None, "stderr": None, "trace": None},
    }
