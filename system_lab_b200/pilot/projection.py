"""PROJECTION stage helper: fit the execution model from a few micro-config runs.

``T_step = T_comp + T_comm_exposed + T_bubble`` with ``T_comp = a * mbs + b`` fitted from short single-node
runs at different micro-batch sizes (``skills/pilot/workflow/projection.md:40-86``,
``skills/pilot/execution-model/SKILL.md:28-63``); memory comes from the analytic model in
``constraints.estimate_memory``.  Confidence is the share of runs that completed.
"""
from __future__ import annotations

import copy

from . import policy


def fit_linear(xs, ys):
    n = len(xs)
    if n == 0:
        return None
    if n == 1:
        return {"a": ys[0] / max(xs[0], 1), "b": 0.0}
    mx, my = sum(xs) / n, sum(ys) / n
    var = sum((x - mx) ** 2 for x in xs)
    a = sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / var if var else 0.0
    return {"a": a, "b": my - a * mx}


def profile_micro_configs(ctx, configs: dict) -> dict:
    base = configs.get("base_plan") or policy.default_plan(ctx.world)
    mbs_values = configs.get("mbs", [1, 2])
    steps = int(configs.get("steps", 8))
    runs, xs, ys = [], [], []
    for mbs in mbs_values:
        plan = copy.deepcopy(base)
        plan["id"] = f"proj_mbs{mbs}"
        plan["runtime"]["mbs"] = mbs
        plan["runtime"]["gbs"] = mbs * plan["parallelism"]["dp"]
        snap = ctx.runner.wait(ctx.runner.submit(plan, steps, mode="projection"))
        ms = (snap.get("metrics") or {}).get("step_time_ms")
        runs.append({"mbs": mbs, "status": snap["status"], "step_time_ms": ms,
                     "mem_peak_gb": (snap.get("metrics") or {}).get("mem_peak_gb")})
        if snap["status"] == "ok" and ms:
            xs.append(mbs)
            ys.append(ms)
    fit = fit_linear(xs, ys)
    return {"runs": runs, "fit": {"t_comp_ms": fit} if fit else None,
            "confidence": len(xs) / max(len(mbs_values), 1),
            "bubble_model": "(pp-1)/(pp-1+M*V)", "mem_model": "constraints.estimate_memory"}
