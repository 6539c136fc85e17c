"""REPORT stage: what a tuning session found, built from the state directory only.

Contents follow ``skills/workflow/report.md`` (reference: ``skills/pilot/workflow/report.md``): outcome and budget,
champion vs baseline, the path round by round, dead ends with reasons, levers not tried, how to reproduce.  Every
number is read from a Snapshot or another artifact; a failed session still gets a report.
"""
from __future__ import annotations

import json
from pathlib import Path

from . import policy


def _load(store, kind: str, default=None):
    p = store.latest_artifact(kind)
    return json.loads(p.read_text()) if p else default


def _all(store, kind: str) -> list:
    return [json.loads(p.read_text()) for p in sorted(store.artifact_dir.glob(f"*_{kind}_*"))]


def _plan_diff(a: dict, b: dict) -> dict:
    out = {}
    for sec in ("parallelism", "runtime", "precision", "comm", "moe"):
        for k, v in (b.get(sec) or {}).items():
            if (a.get(sec) or {}).get(k) != v:
                out[f"{sec}.{k}"] = {"from": (a.get(sec) or {}).get(k), "to": v}
    ea, eb = (a.get("env") or {}).get("diff", {}), (b.get("env") or {}).get("diff", {})
    for k in sorted(set(ea) | set(eb)):
        if ea.get(k) != eb.get(k):
            out[f"env.{k}"] = {"from": ea.get(k), "to": eb.get(k)}
    return out


def build_report(store, state) -> dict:
    graph = policy.PlanGraph.from_dict(_load(store, "PlanGraph", {}) or {})
    nodes = graph.nodes
    base = nodes.get("r0_p0")
    champ = nodes.get(graph.champion) if graph.champion else None
    champ_snap = _load(store, "ChampionSnapshot")
    base_tps = (base or {}).get("tps")
    champ_tps = (champ or {}).get("tps")
    used, total = state.budget_used.model_dump(), state.budget_total.model_dump()
    rounds = {}
    for pid, n in nodes.items():
        r = pid.split("_")[0]
        rounds.setdefault(r, []).append({"plan": pid, "axis": n.get("derived_axis"), "status": n.get("status"),
                                         "tps": n.get("tps"), "parent": n["plan"].get("parent")})
    diagnoses = [{"bottleneck": d.get("bottleneck"), "fired": (d.get("fired_rules") or [])[:2],
                  "confidence": d.get("confidence")} for d in _all(store, "DiagnosisReport")]
    tried = {n.get("derived_axis") for n in nodes.values()}
    last_b = diagnoses[-1]["bottleneck"] if diagnoses else "COMPUTE"
    not_tried = [l["axis"] for l in policy.LEVERS.get(last_b, []) if l["axis"] not in tried]
    job_cmd = None
    if champ_snap and champ_snap.get("job_id"):
        p = store.jobs_dir / champ_snap["job_id"] / "cmd.json"
        if p.exists():
            job_cmd = json.loads(p.read_text()).get("cmd")
    return {
        "session": state.session_id,
        "outcome": {"stop_reason": state.stop_reason, "final_stage": state.current_stage.value, "rounds": state.round_id,
                    "budget_used": used, "budget_total": total, "failure_counts": dict(state.failure_counts)},
        "champion": {"plan_id": graph.champion, "tps": champ_tps, "baseline_tps": base_tps,
                     "gain_vs_baseline_pct": (100.0 * (champ_tps / base_tps - 1.0)) if (champ_tps and base_tps) else None,
                     "step_time_ms": ((champ_snap or {}).get("metrics") or {}).get("step_time_ms"),
                     "mem_peak_gb": ((champ_snap or {}).get("metrics") or {}).get("mem_peak_gb"),
                     "diff_vs_baseline": _plan_diff(base["plan"], champ["plan"]) if (base and champ) else {},
                     "plan": champ["plan"] if champ else None},
        "path": {"rounds": rounds, "diagnoses": diagnoses,
                 "settle": [{k: d.get(k) for k in ("promoted", "champion", "gain_vs_previous", "dead", "stop")}
                            for d in _all(store, "SettleDecision")]},
        "dead_ends": dict(graph.exhausted_neighborhoods) | {
            pid: "dead" for pid, n in nodes.items() if n.get("status") == "dead"},
        "not_tried": not_tried,
        "reproduce": {"command": job_cmd, "snapshot": str(store.latest_artifact("ChampionSnapshot") or "")},
    }


def to_markdown(rep: dict) -> str:
    o, c = rep["outcome"], rep["champion"]
    lines = [f"# Tuning report — session {rep['session']}", "",
             f"**Outcome**: {o['stop_reason'] or o['final_stage']} after {o['rounds']} round(s); GPU-hours "
             f"{o['budget_used'].get('gpu_h', 0):.3f} of {o['budget_total'].get('gpu_h', 0)}, tokens "
             f"{o['budget_used'].get('total_tokens', 0)} of {o['budget_total'].get('total_tokens', 0)}.", ""]
    if c["plan_id"]:
        gain = f"{c['gain_vs_baseline_pct']:+.1f} %" if c["gain_vs_baseline_pct"] is not None else "n/a"
        lines += [f"**Champion** `{c['plan_id']}`: {c['tps'] or 0:,.0f} tokens/s vs baseline {c['baseline_tps'] or 0:,.0f} ({gain}); "
                  f"step {c['step_time_ms'] or 0:.1f} ms, peak memory {c['mem_peak_gb'] or 0:.1f} GB.", ""]
        if c["diff_vs_baseline"]:
            lines += ["| knob | baseline | champion |", "|---|---|---|"]
            lines += [f"| `{k}` | {v['from']} | {v['to']} |" for k, v in c["diff_vs_baseline"].items()]
            lines.append("")
    else:
        lines += ["No champion: the session ended before a baseline completed.", ""]
    lines += ["## Path", "", "| round | plan | derived from | axis | status | tokens/s |", "|---|---|---|---|---|---|"]
    for r, plans in sorted(rep["path"]["rounds"].items()):
        for p in plans:
            tps = f"{p['tps']:,.0f}" if p["tps"] else "-"
            lines.append(f"| {r} | `{p['plan']}` | {p['parent'] or '-'} | {p['axis'] or 'baseline'} | {p['status']} | {tps} |")
    if rep["path"]["diagnoses"]:
        lines += ["", "Diagnoses: " + "; ".join(f"{d['bottleneck']} ({', '.join(d['fired']) or 'fall-through'})"
                                                for d in rep["path"]["diagnoses"])]
    if rep["dead_ends"]:
        lines += ["", "## Dead ends", ""] + [f"* `{k[:80]}`: {v}" for k, v in list(rep["dead_ends"].items())[:20]]
    if rep["not_tried"]:
        lines += ["", "## Not tried", "", ", ".join(f"`{a}`" for a in rep["not_tried"])]
    if rep["reproduce"]["command"]:
        lines += ["", "## Reproduce", "", "```", " ".join(rep["reproduce"]["command"]), "```"]
    return "\n".join(lines) + "\n"


def write_report(store, state) -> Path:
    rep = build_report(store, state)
    store.write_artifact("TuningReport", "report.json", json.dumps(rep, indent=2, default=str))
    art = store.write_artifact("TuningReport", "report.md", to_markdown(rep))
    return Path(art.ref)
