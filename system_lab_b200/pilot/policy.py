"""Executable form of the tuner's skill pack: diagnosis rules, re-planning, loss comparison, early stop and
settle logic.  The reference ships these as prose contracts for an LLM worker
(``skills/pilot/workflow/{diagnose,replan,correctness,execute,settle,execution_strategy}.md``); here they are
plain functions so a whole tuning session can run deterministically (``--backend rules``) and so an LLM
worker's decisions can be checked against them.

Thresholds (single-node values; all from the reference's skill pack):

* MEMORY     : OOM event, peak > 0.92 HBM, or reserved/allocated > 1.4          (diagnose.md:45-117, oom.md:36-89)
* MOE        : expert load imbalance > 25 %
* PIPELINE   : bubble ratio > 0.15
* COMM       : exposed comm ratio > 0.20 (0.25 multi-node)
* COMPUTE    : otherwise (utilisation < 0.65 or tps < 0.8 x expected are its soft signals)
* promote    : challenger tps > champion x 1.02 (settle.md:30-60); hard win 1.05
* early stop : tps < 0.85 x champion after 50 steps, < 0.70 x predicted, loss drift > 5 % at step 100, NaN,
               memory > 0.97 HBM, no progress for 300 s (execute.md:85-101)
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any

HBM_GB = 180.0
MEM_SAFE, MEM_IMMINENT, FRAG_RATIO = 0.92, 0.97, 1.4
IMBALANCE_PCT, BUBBLE_MAX, COMM_SINGLE, COMM_MULTI = 25.0, 0.15, 0.20, 0.25
UTIL_MIN, TPS_VS_EXPECTED = 0.65, 0.80
EPS_PROMOTE, EPS_HARD = 0.02, 0.05
EARLY_TPS_CHAMPION, EARLY_TPS_PREDICTED, EARLY_LOSS_DRIFT = 0.85, 0.70, 0.05
HANG_TIMEOUT_S = 300.0
NOVELTY_BONUS, STABILITY_BONUS = 1.2, 1.1

# ordered levers per bottleneck: (axis, candidate values or transform, expected gain %, relative cost, note)
LEVERS: dict[str, list[dict]] = {
    "COMPUTE": [
        {"axis": "runtime.mbs", "op": "double", "gain": 8.0, "risk": "memory"},
        {"axis": "runtime.recompute", "op": "relax", "gain": 10.0, "risk": "memory"},
        {"axis": "parallelism.tp", "op": "halve", "gain": 6.0, "needs": "tp>1",
         "note": "fewer exposed all-reduces per layer, larger GEMMs per rank"},
        {"axis": "parallelism.vpp", "op": "set", "values": [2], "gain": 3.0, "needs": "pp>1"},
        {"axis": "precision.fp8", "op": "set", "values": [True], "gain": 20.0, "risk": "numeric"},
    ],
    "MEMORY": [
        {"axis": "runtime.recompute", "op": "tighten", "gain": 0.0, "mem": -0.4},
        {"axis": "precision.optimizer_state_dtype", "op": "set", "values": ["bf16", "fp8"], "gain": 0.0, "mem": -0.3},
        {"axis": "runtime.mbs", "op": "halve", "gain": -5.0, "mem": -0.3},
        {"axis": "parallelism.ep", "op": "double", "gain": -2.0, "mem": -0.3},
        {"axis": "runtime.optimizer_in_backward", "op": "set", "values": [True], "gain": 0.0, "mem": -0.15},
        {"axis": "parallelism.tp", "op": "double", "gain": -8.0, "mem": -0.3,
         "note": "last resort: splits attention activations and the MoE rows of a rank; two exposed collectives per layer"},
        {"axis": "parallelism.sp", "op": "set", "values": [True], "gain": 0.0, "mem": -0.1, "needs": "tp>1",
         "note": "sequence parallelism: norms and residual stream on 1/tp of every sequence (SP requires TP > 1)"},
    ],
    "COMM": [
        {"axis": "comm.dispatcher", "op": "set", "values": ["fused"], "gain": 15.0},
        {"axis": "comm.fsdp_fused_collectives", "op": "set", "values": [True], "gain": 4.0},
        {"axis": "parallelism.tp", "op": "halve", "gain": 8.0, "needs": "tp>1", "risk": "memory"},
        {"axis": "parallelism.ep", "op": "halve", "gain": 6.0, "risk": "memory"},
        {"axis": "comm.bucket_size_mb", "op": "set", "values": [64, 160], "gain": 2.0},
        {"axis": "env.NCCL_NVLS_ENABLE", "op": "set", "values": ["1"], "gain": 2.0},
    ],
    "PIPELINE": [
        {"axis": "parallelism.vpp", "op": "set", "values": [2], "gain": 8.0, "needs": "pp>1"},
        {"axis": "runtime.mbs", "op": "halve", "gain": 5.0, "note": "more micro-batches"},
        {"axis": "parallelism.pp", "op": "halve", "gain": 6.0, "risk": "memory"},
    ],
    "MOE_IMBALANCED": [
        {"axis": "moe.expert_relocation_interval", "op": "set", "values": [100], "gain": 12.0,
         "note": "re-place experts on ranks by measured load; the math is unchanged"},
        {"axis": "moe.capacity_factor", "op": "set", "values": [1.25, 2.0], "gain": 3.0},
        {"axis": "moe.aux_loss_coeff", "op": "set", "values": [1e-3, 1e-2], "gain": 5.0},
        {"axis": "moe.load_balancing", "op": "set", "values": ["bias"], "gain": 5.0},
        {"axis": "parallelism.ep", "op": "halve", "gain": 4.0},
    ],
}
CANDIDATE_AXES = {k: [l["axis"] for l in v] for k, v in LEVERS.items()}


# ------------------------------------------------------------------------------------- diagnose
def diagnose(snapshot: dict, *, multi_node: bool = False, expected_tps: float | None = None,
             hbm_gb: float = HBM_GB) -> dict:
    """Top-down bottleneck classification of one Snapshot; first rule that fires wins."""
    m = snapshot.get("metrics", {})
    fired: list[str] = []
    soft: list[str] = []
    if snapshot.get("status") == "oom" or m.get("has_oom_event"):
        fired.append("MEMORY:oom_event")
    mem = m.get("mem_peak_gb") or 0.0
    if mem > MEM_SAFE * hbm_gb:
        fired.append(f"MEMORY:peak {mem:.1f} GB > {MEM_SAFE:.2f} x {hbm_gb:.0f}")
    frag = m.get("mem_reserved_to_alloc_ratio")
    if frag and frag > FRAG_RATIO:
        fired.append(f"MEMORY:fragmentation {frag:.2f} > {FRAG_RATIO}")
    imb = m.get("expert_load_imbalance_pct")
    if imb is not None and imb > IMBALANCE_PCT:
        fired.append(f"MOE_IMBALANCED:{imb:.0f} % > {IMBALANCE_PCT:.0f} %")
    bub = m.get("bubble_ratio")
    if bub is not None and bub > BUBBLE_MAX:
        fired.append(f"PIPELINE:bubble {bub:.2f} > {BUBBLE_MAX}")
    comm = m.get("comm_ratio")
    thr = COMM_MULTI if multi_node else COMM_SINGLE
    if comm is not None and comm > thr:
        fired.append(f"COMM:exposed {comm:.2f} > {thr}")
    util = m.get("gpu_util_avg")
    if util is not None and util < UTIL_MIN:
        soft.append(f"gpu_util {util:.2f} < {UTIL_MIN}")
    tps = m.get("tps")
    if expected_tps and tps and tps < TPS_VS_EXPECTED * expected_tps:
        soft.append(f"tps {tps:.0f} < {TPS_VS_EXPECTED} x expected {expected_tps:.0f}")
    bottleneck = fired[0].split(":")[0] if fired else "COMPUTE"
    low_conf = snapshot.get("confidence_in_metrics") == "low"
    confidence = (0.5 if low_conf else 0.8) if fired else (0.4 if low_conf else 0.6)
    return {"bottleneck": bottleneck, "fired_rules": fired, "soft_signals": soft, "confidence": confidence,
            "candidate_axes": CANDIDATE_AXES[bottleneck],
            "env_suspect": bottleneck == "COMM" and (m.get("overlap_ratio") or 1.0) < 0.3,
            "suggested_strategy": "champion_challenger" if confidence >= 0.6 else "local_sweep"}


# ------------------------------------------------------------------------------------- plans
def default_plan(world: int, *, ep: int | None = None, mbs: int = 2, gbs: int | None = None) -> dict:
    ep = ep or world
    return {"id": "r0_p0", "parent": None,
            "parallelism": {"tp": 1, "pp": 1, "dp": world, "ep": ep, "vpp": 1, "cp": 1, "sp": False},
            "runtime": {"mbs": mbs, "gbs": gbs or mbs * world, "recompute": "full", "optimizer_in_backward": False},
            "precision": {"fp8": False, "optimizer_state_dtype": "fp32", "master_weights": True},
            "comm": {"dispatcher": "fused", "fsdp_fused_collectives": False, "bucket_size_mb": 160},
            "moe": {"capacity_factor": 0.0, "aux_loss_coeff": 0.0, "load_balancing": "aux_loss",
                    "expert_relocation_interval": 0},
            "env": {"diff": {}}}


def plan_to_overrides(plan: dict) -> tuple[list[str], dict[str, str]]:
    """Translate a Plan into trainer ``key=value`` overrides plus the environment diff."""
    p, r, pr, c, mo = plan["parallelism"], plan["runtime"], plan["precision"], plan["comm"], plan["moe"]
    ov = [f"tensor_model_parallel_size={p['tp']}", f"pipeline_model_parallel_size={p['pp']}",
          f"expert_model_parallel_size={p['ep']}", f"virtual_pipeline_model_parallel_size={p['vpp']}",
          f"context_parallel_size={p.get('cp', 1)}", f"sequence_parallel={str(bool(p.get('sp', False))).lower()}",
          f"micro_batch_size={r['mbs']}", f"global_batch_size={r['gbs']}",
          f"recompute_granularity={r['recompute']}", f"optimizer_in_backward={str(r['optimizer_in_backward']).lower()}",
          f"fp8={str(pr['fp8']).lower()}", f"optimizer_state_dtype={pr['optimizer_state_dtype']}",
          f"master_weights={str(pr['master_weights']).lower()}", f"moe_token_dispatcher_type={c['dispatcher']}",
          f"fsdp_fused_collectives={str(c['fsdp_fused_collectives']).lower()}",
          f"ddp_bucket_size={int(c['bucket_size_mb']) * 250_000}", f"moe_capacity_factor={mo['capacity_factor']}",
          f"moe_aux_loss_coeff={mo['aux_loss_coeff']}", f"moe_router_load_balancing_type={mo['load_balancing']}",
          f"moe_expert_relocation_interval={int(mo.get('expert_relocation_interval', 0))}"]
    return ov, {k: str(v) for k, v in plan.get("env", {}).get("diff", {}).items()}


def bubble_ratio(pp: int, microbatches: int, vpp: int = 1) -> float:
    """``(pp-1) / (pp-1 + M*V)`` (``skills/pilot/optimization/pipeline/SKILL.md:19-42``)."""
    return 0.0 if pp <= 1 else (pp - 1) / (pp - 1 + microbatches * vpp)


_RECOMPUTE_ORDER = ["none", "selective", "full"]


def _apply(plan: dict, lever: dict, value: Any) -> dict | None:
    q = copy.deepcopy(plan)
    sec, key = lever["axis"].split(".", 1)
    if sec == "env":
        q["env"]["diff"][key] = value
        return q
    cur = q[sec].get(key, False) if key == "sp" else q[sec][key]
    op = lever["op"]
    if op == "double":
        new = cur * 2
    elif op == "halve":
        if cur <= 1:
            return None
        new = cur // 2
    elif op == "relax":
        i = _RECOMPUTE_ORDER.index(cur)
        if i == 0:
            return None
        new = _RECOMPUTE_ORDER[i - 1]
    elif op == "tighten":
        i = _RECOMPUTE_ORDER.index(cur)
        if i == len(_RECOMPUTE_ORDER) - 1:
            return None
        new = _RECOMPUTE_ORDER[i + 1]
    else:
        new = value
    if new == cur:
        return None
    q[sec][key] = new
    if lever["axis"] == "parallelism.tp":
        # the world size is fixed: a wider tensor-parallel group takes its ranks from the data axis
        dp = q["parallelism"]["dp"] * cur
        if dp % new:
            return None
        q["parallelism"]["dp"] = dp // new
        if new <= 1:
            q["parallelism"]["sp"] = False          # sequence parallelism needs a tensor-parallel group
        if q["runtime"]["gbs"] % (q["runtime"]["mbs"] * q["parallelism"]["dp"]):
            return None
    if lever["axis"] == "runtime.mbs":
        dp = q["parallelism"]["dp"]
        if q["runtime"]["gbs"] % (new * dp):
            return None
    return q


def priority(gain_pct: float, confidence: float, cost_gpu_h: float, novel: bool, parent_stable: bool) -> float:
    """``max(gain,0.1) * confidence / max(cost,0.05) * novelty * parent_stability`` (``pilot/README.v2.md:859-863``)."""
    return (max(gain_pct, 0.1) * confidence / max(cost_gpu_h, 0.05)
            * (NOVELTY_BONUS if novel else 1.0) * (STABILITY_BONUS if parent_stable else 1.0))


def replan(champion: dict, diagnosis: dict, graph: "PlanGraph", *, check, estimate_mem, round_id: int,
           top_k: int = 3, cost_gpu_h: float = 0.05, explore: bool = False) -> list[dict]:
    """One candidate per (source, axis, value); filtered by legality, the 92 % memory rule and exhausted
    neighbourhoods; ranked by priority.  ``check(plan) -> list[violations]``, ``estimate_mem(plan) -> GB``."""
    sources = [champion] + ([graph.nodes[i]["plan"] for i in graph.shelved()[:2]] if explore else [])
    levers = list(LEVERS[diagnosis["bottleneck"]])
    if explore:
        levers += [l for b, ls in LEVERS.items() if b != diagnosis["bottleneck"] for l in ls[:1]]
    cands = []
    for src in sources:
        for lever in levers:
            if lever.get("needs") == "pp>1" and src["parallelism"]["pp"] <= 1:
                continue
            if lever.get("needs") == "tp>1" and src["parallelism"].get("tp", 1) <= 1:
                continue
            for value in lever.get("values", [None]):
                q = _apply(src, lever, value)
                if q is None:
                    continue
                key = graph.signature(q)
                if graph.exhausted(key):
                    continue
                if check(q):
                    graph.mark_exhausted(key, "constraint_violation")
                    continue
                mem = estimate_mem(q)
                if mem > MEM_SAFE * HBM_GB:
                    graph.mark_exhausted(key, f"estimated memory {mem:.0f} GB")
                    continue
                cands.append({"plan": q, "axis": lever["axis"], "value": q[lever["axis"].split(".")[0]].get(
                    lever["axis"].split(".", 1)[1], value), "predicted_gain_pct": lever["gain"], "est_mem_gb": mem,
                    "priority": priority(lever["gain"], diagnosis["confidence"], cost_gpu_h,
                                         novel=not graph.seen_axis(lever["axis"]), parent_stable=src is champion),
                    "parent": src["id"]})
    cands.sort(key=lambda c: -c["priority"])
    out = cands[:top_k]
    for i, c in enumerate(out):
        c["plan"]["id"] = f"r{round_id}_p{i}"
        c["plan"]["parent"] = c["parent"]
    return out


# ------------------------------------------------------------------------------------- plan graph
@dataclass
class PlanGraph:
    """Search bookkeeping (``skills/pilot/workflow/plan_graph.md:19-135``): node status, derivation axis,
    exhausted neighbourhoods with reasons, counters."""
    nodes: dict[str, dict] = field(default_factory=dict)
    exhausted_neighborhoods: dict[str, str] = field(default_factory=dict)
    champion: str | None = None
    rounds_without_gain: int = 0

    @staticmethod
    def signature(plan: dict) -> str:
        keep = {k: plan[k] for k in ("parallelism", "runtime", "precision", "comm", "moe")}
        keep["env"] = plan.get("env", {}).get("diff", {})
        return repr(sorted((k, sorted(v.items())) for k, v in keep.items()))

    def add(self, plan: dict, status: str = "pending", axis: str | None = None) -> None:
        self.nodes[plan["id"]] = {"plan": plan, "status": status, "derived_axis": axis, "tps": None}

    def exhausted(self, sig: str) -> bool:
        return sig in self.exhausted_neighborhoods or any(self.signature(n["plan"]) == sig for n in self.nodes.values())

    def mark_exhausted(self, sig: str, reason: str) -> None:
        self.exhausted_neighborhoods[sig] = reason

    def seen_axis(self, axis: str) -> bool:
        return any(n["derived_axis"] == axis for n in self.nodes.values())

    def shelved(self) -> list[str]:
        s = [(n["tps"] or 0.0, i) for i, n in self.nodes.items() if n["status"] == "shelved"]
        return [i for _, i in sorted(s, reverse=True)]

    def to_dict(self) -> dict:
        return {"nodes": self.nodes, "exhausted_neighborhoods": self.exhausted_neighborhoods,
                "champion": self.champion, "rounds_without_gain": self.rounds_without_gain}

    @staticmethod
    def from_dict(d: dict) -> "PlanGraph":
        return PlanGraph(d.get("nodes", {}), d.get("exhausted_neighborhoods", {}), d.get("champion"),
                         d.get("rounds_without_gain", 0))


# ------------------------------------------------------------------------------------- correctness
def _ema(xs, alpha=0.1):
    out, cur = [], None
    for x in xs:
        cur = x if cur is None else alpha * x + (1 - alpha) * cur
        out.append(cur)
    return out


def compare_loss(cur_curve, ref_curve, *, tolerance: float = 0.01, lite: bool = False) -> dict:
    """Align two ``[[step, loss], ...]`` curves on common steps, smooth with EMA(0.1) and take the largest
    relative gap.  Full gate: <= tolerance over >= 200 steps; lite gate: <= 2 x tolerance over >= 100 steps
    (``skills/pilot/workflow/correctness.md:62-96``).  NaN anywhere fails outright."""
    cur, ref = dict(map(tuple, cur_curve)), dict(map(tuple, ref_curve))
    steps = sorted(set(cur) & set(ref))
    if any(not math.isfinite(cur[s]) for s in cur):
        return {"pass": False, "delta_pct": None, "reason": "NaN/Inf in loss curve", "steps_compared": len(steps)}
    if not steps:
        return {"pass": False, "delta_pct": None, "reason": "no common steps", "steps_compared": 0}
    ec, er = _ema([cur[s] for s in steps]), _ema([ref[s] for s in steps])
    delta = max(abs(a - b) / max(abs(b), 1e-12) for a, b in zip(ec, er))
    need = 100 if lite else 200
    limit = tolerance * (2 if lite else 1)
    span = steps[-1] - steps[0] + 1
    ok = delta <= limit
    return {"pass": ok, "delta_pct": 100 * delta, "limit_pct": 100 * limit, "steps_compared": len(steps),
            "enough_steps": span >= need,
            "reason": "" if ok else f"EMA loss gap {100 * delta:.2f} % > {100 * limit:.2f} %"}


# ------------------------------------------------------------------------------------- execute / settle
def early_stop(partial: dict, *, champion_tps: float | None, predicted_tps: float | None,
               ref_loss_at_100: float | None = None, min_steps: int = 20, hbm_gb: float = HBM_GB) -> str | None:
    """Reason to kill a running job early, or None (``skills/pilot/workflow/execute.md:85-101``)."""
    steps = partial.get("completed_steps", 0)
    if partial.get("has_nan"):
        return "nan"
    if (partial.get("mem_peak_gb") or 0) > MEM_IMMINENT * hbm_gb:
        return "oom_imminent"
    if partial.get("seconds_since_progress", 0) > HANG_TIMEOUT_S:
        return "hang_5min"
    if steps < min_steps:
        return None
    tps = partial.get("tps")
    if tps and champion_tps and steps >= 50 and tps < EARLY_TPS_CHAMPION * champion_tps:
        return "tps_below_champion_85pct"
    if tps and predicted_tps and tps < EARLY_TPS_PREDICTED * predicted_tps:
        return "tps_below_prediction_70pct"
    loss = partial.get("loss")
    if ref_loss_at_100 and loss and steps >= 100 and abs(loss - ref_loss_at_100) / abs(ref_loss_at_100) > EARLY_LOSS_DRIFT:
        return "loss_drift_early"
    return None


def settle(graph: PlanGraph, results: list[dict], *, max_stagnant_rounds: int = 2) -> dict:
    """Promote the best challenger if it beats the champion by EPS_PROMOTE, shelve the rest, track stagnation.
    ``results``: ``[{plan_id, tps, status, correctness_ok}]``.  Returns the decision record."""
    champ = graph.nodes.get(graph.champion) if graph.champion else None
    champ_tps = (champ or {}).get("tps") or 0.0
    best = None
    for r in results:
        node = graph.nodes[r["plan_id"]]
        node["tps"] = r.get("tps")
        if r.get("status") != "ok" or not r.get("correctness_ok", True):
            node["status"] = "dead"
            continue
        node["status"] = "shelved"
        if best is None or (r["tps"] or 0) > (best["tps"] or 0):
            best = r
    promoted = False
    if best is not None and (best["tps"] or 0) > champ_tps * (1 + EPS_PROMOTE):
        if champ is not None:
            champ["status"] = "shelved"
        graph.nodes[best["plan_id"]]["status"] = "champion"
        graph.champion = best["plan_id"]
        graph.rounds_without_gain = 0
        promoted = True
    else:
        graph.rounds_without_gain += 1
    dead = sum(1 for r in results if graph.nodes[r["plan_id"]]["status"] == "dead")
    gain = ((best["tps"] / champ_tps - 1) if (best and champ_tps) else None)
    stop = None
    if graph.rounds_without_gain >= max_stagnant_rounds + 1:
        stop = "STAGNATION"
    return {"promoted": promoted, "champion": graph.champion, "gain_vs_previous": gain,
            "hard_win": bool(gain is not None and gain > EPS_HARD), "dead": dead,
            "explore_next": graph.rounds_without_gain >= max_stagnant_rounds or (results and dead / len(results) > 0.5),
            "stop": stop}


def classify_failure(exit_code: int, log_tail: str, timed_out: bool) -> str:
    """Map a failed job to a failure kind, most specific first: NUMERICAL > OOM > HANG > ... > UNKNOWN
    (``skills/pilot/constraints/validation.md:28-147``)."""
    t = log_tail.lower()
    if "numericalerror" in t or "nan" in t and "loss" in t:
        return "NUMERICAL"
    if "out of memory" in t or "cuda oom" in t or "outofmemoryerror" in t:
        return "OOM"
    if timed_out or "devicehang" in t or "timeout" in t or "watchdog" in t:
        return "HANG" if not timed_out else "TIMEOUT"
    if "configerror" in t or "not divisible" in t or "unknown config key" in t:
        return "CONSTRAINT_VIOLATION"
    if exit_code != 0:
        return "TOOL_ERROR"
    return "UNKNOWN"
