"""VRAM health of a training run: allocator counters -> verdict, and a bucket decomposition of the peak.

Two questions a run's memory numbers must answer before a config is kept: *how close to the cap is the
driver-side reservation* (what ``nvidia-smi`` shows and what OOMs), and *what is the peak made of*.  The
counters are the ones ``torch.cuda.memory_stats`` exposes; the decomposition is the analytic model the tuner
uses (``pilot/constraints.py``) laid out as named buckets so the sum can be reconciled against the measured
peak.  If more than 10 % of the peak is unaccounted the estimate is wrong and the table says so.

Reference behaviour: ``.cursor/skills/trace-vram-canvas/SKILL.md:176-237`` (fields ``current/pmax/rmax/
retires/capGB``; derived reserved %, allocated %, fragmentation %, headroom; TIGHT at 95-98 % reserved,
CRITICAL at 98 %; bucket sets A (adapter fine-tune), B (full training), C (MoE pretraining); the 10 % rule).
"""
from __future__ import annotations

import argparse
import json
from dataclasses import asdict, dataclass, field
from typing import Any

GB = 1e9


@dataclass
class VramSample:
    current_gb: float        # allocated at the sample point
    pmax_gb: float           # peak allocated across the run
    rmax_gb: float           # peak reserved by the caching allocator (driver-side footprint)
    retires: int             # allocation retries after a cache flush: any value > 0 is allocator pressure
    cap_gb: float            # device memory


def sample_device(device=None) -> VramSample:
    """Read the counters of ``device`` (default: current CUDA device)."""
    import torch
    st = torch.cuda.memory_stats(device)
    props = torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device())
    return VramSample(current_gb=st.get("allocated_bytes.all.current", 0) / GB,
                      pmax_gb=st.get("allocated_bytes.all.peak", 0) / GB,
                      rmax_gb=st.get("reserved_bytes.all.peak", 0) / GB,
                      retires=int(st.get("num_alloc_retries", 0)),
                      cap_gb=props.total_memory / GB)


def health(s: VramSample) -> dict:
    """Derived ratios and the verdict.  ``frag_pct`` is the share of the reservation that is cache slack."""
    cap = max(s.cap_gb, 1e-9)
    reserved_pct = 100.0 * s.rmax_gb / cap
    alloc_pct = 100.0 * s.pmax_gb / cap
    frag_pct = 100.0 * max(s.rmax_gb - s.pmax_gb, 0.0) / max(s.rmax_gb, 1e-9)
    if reserved_pct >= 98.0:
        verdict = "CRITICAL"
    elif reserved_pct >= 95.0:
        verdict = "TIGHT"
    elif s.retires > 0:
        verdict = "PRESSURE"          # fits, but the allocator had to flush its cache to get there
    else:
        verdict = "OK"
    return {"reserved_pct": reserved_pct, "alloc_pct": alloc_pct, "frag_pct": frag_pct,
            "headroom_gb": s.cap_gb - s.rmax_gb, "retires": s.retires, "verdict": verdict}


@dataclass
class Buckets:
    mode: str
    rows: list = field(default_factory=list)      # [{"bucket": str, "gb": float, "how": str}]
    pmax_gb: float = 0.0
    unaccounted_gb: float = 0.0
    unaccounted_pct: float = 0.0
    consistent: bool = True

    def to_dict(self) -> dict:
        return asdict(self)


def pick_mode(cfg: Any, trainable_fraction: float = 1.0) -> str:
    """A = adapter fine-tune (few trainable parameters), B = full training of a dense model, C = MoE."""
    if trainable_fraction < 0.05:
        return "A"
    return "C" if cfg.model.num_experts > 0 else "B"


def decompose(cfg: Any, world: int, sample: VramSample | None = None, trainable_fraction: float = 1.0,
              mode: str | None = None) -> Buckets:
    """Bucket table for ``cfg`` on ``world`` GPUs; reconciled against ``sample.pmax_gb`` when given."""
    from ..pilot.constraints import estimate_memory, param_counts
    pc = param_counts(cfg.model)
    if trainable_fraction >= 1.0 and pc.get("lora"):
        trainable_fraction = pc["trainable"] / max(pc["total"], 1)      # LoRA: only the adapters train
    mode = mode or pick_mode(cfg, trainable_fraction)
    est = estimate_memory(cfg, world)
    pr, par = cfg.precision, cfg.parallel
    pp = max(par.pipeline_model_parallel_size, 1)
    dp = max(world // (pp * max(par.context_parallel_size, 1)), 1)
    ep = max(min(par.expert_model_parallel_size, dp), 1)
    wbytes = 2 if pr.params_dtype == "bf16" else 4
    shard_dense = dp if par.fsdp else 1
    shard_exp = max(dp // ep, 1) if par.fsdp else 1
    dense_p = (pc["total"] - pc["experts"]) / pp
    exp_p = pc["experts"] / pp / ep
    state_b = {"fp32": 8, "bf16": 4, "fp8": 2}[pr.optimizer_state_dtype]
    master_b = 4 if (pr.params_dtype != "fp32" and pr.master_weights) else 0
    nmb = max(cfg.train.global_batch_size // max(cfg.train.micro_batch_size * dp, 1), 1)
    grad_b = 0 if cfg.train.optimizer_in_backward else (2 if (wbytes == 2 and nmb <= 1) else 4)
    tf = trainable_fraction
    rows = []

    def add(name, nbytes, how):
        rows.append({"bucket": name, "gb": nbytes / GB, "how": how})

    if mode == "C":
        add("Dense weights", dense_p * wbytes / shard_dense, f"{dense_p / 1e9:.2f} B params x {wbytes} B / {shard_dense}")
        add("MoE expert weights", exp_p * wbytes / shard_exp,
            f"{pc["experts"] / 1e9:.2f} B params / pp{pp} / ep{ep} x {wbytes} B / {shard_exp}")
        add("Optimizer state + master + grads (sharded)",
            (dense_p / shard_dense + exp_p / shard_exp) * (state_b + master_b + grad_b),
            f"({state_b} moments + {master_b} master + {grad_b} grad) B per sharded param")
    elif mode == "B":
        add("Weights", (dense_p / shard_dense + exp_p / shard_exp) * wbytes, f"{wbytes} B per sharded param")
        add("Master copy", (dense_p / shard_dense + exp_p / shard_exp) * master_b, f"{master_b} B per sharded param")
        add("Adam state (m + v)", (dense_p / shard_dense + exp_p / shard_exp) * state_b, f"{state_b} B per sharded param")
        add("Gradients", (dense_p / shard_dense + exp_p / shard_exp) * grad_b, f"{grad_b} B per sharded param")
    else:                                             # A: frozen base weights, tiny trainable set
        add("Weights (frozen base)", (dense_p / shard_dense + exp_p / shard_exp) * wbytes, f"{wbytes} B per param")
        add("Adapter grads + Adam state", (dense_p + exp_p) * tf * (grad_b + state_b + master_b) / dp,
            f"trainable fraction {tf:.4f}")
    acts = est.get("activation_bytes", 0.0)
    add("Activations" + (" + token-permute buffers" if mode == "C" else ""), acts,
        f"recompute={pr.recompute_granularity}, micro-batch {cfg.train.micro_batch_size} x seq {cfg.model.seq_length}")
    work = est.get("transient_bytes", 0.0) + est.get("logits_bytes", 0.0)
    add("Gathered layer / dispatch buffers / loss chunk", work,
        "un-sharded layer in flight, peer-memory dispatch buffers, logits of one loss chunk")
    total = sum(r["gb"] for r in rows)
    b = Buckets(mode=mode, rows=rows)
    if sample is not None:
        add("Allocator slack (reserved - allocated)", max(sample.rmax_gb - sample.pmax_gb, 0.0) * GB, "computed")
        b.pmax_gb = sample.pmax_gb
        b.unaccounted_gb = sample.pmax_gb - total
        b.unaccounted_pct = 100.0 * abs(b.unaccounted_gb) / max(sample.pmax_gb, 1e-9)
        b.consistent = b.unaccounted_pct <= 10.0
        rows.append({"bucket": "Other / unaccounted", "gb": b.unaccounted_gb, "how": "peak allocated - sum of the model rows"})
    return b


def format_table(h: dict, b: Buckets) -> str:
    out = [f"VRAM verdict {h['verdict']}: reserved {h['reserved_pct']:.1f} %, allocated {h['alloc_pct']:.1f} %, "
           f"fragmentation {h['frag_pct']:.1f} %, headroom {h['headroom_gb']:.1f} GB, retries {h['retires']}",
           f"bucket decomposition (mode {b.mode}):"]
    for r in b.rows:
        out.append(f"  {r['bucket']:46s} {r['gb']:8.2f} GB   {r['how']}")
    if b.pmax_gb and not b.consistent:
        out.append(f"  WARNING: {b.unaccounted_pct:.0f} % of the peak is unaccounted - the estimate is wrong")
    return "\n".join(out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="VRAM verdict and bucket table from counters + a config")
    ap.add_argument("--preset", default=None)
    ap.add_argument("--config", default=None)
    ap.add_argument("--world", type=int, default=1)
    ap.add_argument("--current", type=float, default=0.0)
    ap.add_argument("--pmax", type=float, required=True, help="peak allocated, GB")
    ap.add_argument("--rmax", type=float, required=True, help="peak reserved, GB")
    ap.add_argument("--retires", type=int, default=0)
    ap.add_argument("--cap", type=float, default=192.3, help="device memory, GB (B200: 183 359 MiB)")
    ap.add_argument("--json", default="")
    ap.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    from ..config import Config
    cfg = Config.load(a.config, a.overrides, a.preset)
    s = VramSample(a.current, a.pmax, a.rmax, a.retires, a.cap)
    h, b = health(s), decompose(cfg, a.world, s)
    print(format_table(h, b))
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"sample": asdict(s), "health": h, "buckets": b.to_dict()}, f, indent=2)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
