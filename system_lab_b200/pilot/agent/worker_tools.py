"""Worker tool schemas (Anthropic tool format) and their handlers.

Thirteen tools — two protocol tools (``return_subagent_result``, ``write_artifact``) and eleven business
tools — with the names, arguments and per-stage scoping of the reference
(``pilot/agent/worker_tools.py:19-256``).  There the business handlers are stubs returning ``STUB:*``
references; here each one does its job against this framework: ``preflight_run`` measures the machine,
``submit_run`` / ``observe_snapshot`` launch and watch the trainer, the ``constraint_*`` tools run the same
legality and memory model the trainer uses, ``observe_compare_loss`` applies the EMA gate, and
``knowledge_write`` appends de-duplicated entries to the knowledge file.
"""
from __future__ import annotations

import json
import time
from pathlib import Path
from typing import Any

from .. import policy
from ..constraints import check_config, estimate_memory
from .schemas import Stage


def _tool(name: str, description: str, properties: dict, required: list[str]) -> dict:
    return {"name": name, "description": description,
            "input_schema": {"type": "object", "properties": properties, "required": required}}


_S, _O, _I = {"type": "string"}, {"type": "object"}, {"type": "integer"}

RETURN_SUBAGENT_RESULT = _tool(
    "return_subagent_result",
    "Return the final SubagentResult to the orchestrator. Call exactly once, last. `summary` is capped at "
    "about 1200 characters (headline + key_metrics); heavy detail goes to write_artifact and is referenced here.",
    {"status": {"type": "string", "enum": ["success", "failed", "escalate"]},
     "artifacts": {"type": "array", "default": [],
                   "items": {"type": "object", "required": ["kind", "ref"],
                             "properties": {"kind": _S, "ref": _S, "size_bytes": _I}}},
     "summary": {"type": "object", "description": "headline + key_metrics, under ~200 tokens"},
     "suggested_transition": {"type": "object", "properties": {"to": _S, "reason": _S}},
     "failure": {"type": "object", "properties": {"kind": _S, "message": _S,
                                                  "escalate_to_orchestrator": {"type": "boolean"}}}},
    ["status", "summary"])
WRITE_ARTIFACT = _tool(
    "write_artifact",
    "Persist a heavy artifact (PlanGraph, CandidatePool, Snapshot, DiagnosisReport, EnvSweepResult, ...) in the "
    "state layer; returns a ref for SubagentResult.artifacts.",
    {"kind": _S, "name": _S, "content": {"type": "string", "description": "YAML or JSON text"}},
    ["kind", "name", "content"])
PREFLIGHT_RUN = _tool("preflight_run", "Measure the hardware baseline; returns a ClusterProfile ref.",
                      {"cluster_id": _S}, ["cluster_id"])
ENV_PROBE_RUN = _tool("env_probe_run", "Validate candidate environment flags with a one-step boot each.",
                      {"cluster_id": _S, "candidate_envs": _O}, ["cluster_id"])
ENV_PROBE_SWEEP = _tool("env_probe_sweep", "Inner-loop sweep: structure fixed, environment diff varied.",
                        {"base_plan_ref": _S, "candidate_envs": _O, "max_steps": {"type": "integer", "default": 50}},
                        ["base_plan_ref", "candidate_envs"])
PROFILER_RUN = _tool("profiler_run", "Single-node profiling of micro-configs; returns a ProfilingResult ref.",
                     {"model_spec": _O, "configs": _O}, ["model_spec", "configs"])
SUBMIT_RUN = _tool("submit_run", "Submit a training job for a plan; returns job_id.  `overrides`: extra trainer "
                   "key=value strings for this job only (a smoke run shrinks the model with them).",
                   {"plan_ref": _S, "cluster_id": _S, "max_steps": _I, "overrides": {"type": "array", "items": _S}},
                   ["plan_ref", "cluster_id"])
OBSERVE_SNAPSHOT = _tool("observe_snapshot", "Collect the job's runtime metrics; returns a Snapshot ref.",
                         {"job_id": _S}, ["job_id"])
OBSERVE_COMPARE_LOSS = _tool("observe_compare_loss", "Correctness gate: compare a job's loss curve with a reference.",
                             {"job_id": _S, "reference_curve_ref": _S}, ["job_id", "reference_curve_ref"])
CONSTRAINT_CHECK = _tool("constraint_check", "Validate a plan's configuration legality.", {"plan_ref": _S}, ["plan_ref"])
CONSTRAINT_CHECK_ENV = _tool("constraint_check_env", "Validate an environment combination (mutex / dangerous flags).",
                             {"env_diff": _O, "baseline": _S}, ["env_diff"])
CONSTRAINT_ESTIMATE_MEM = _tool("constraint_estimate_mem", "Estimate per-GPU memory of a plan.", {"plan_ref": _S},
                                ["plan_ref"])
KNOWLEDGE_WRITE = _tool("knowledge_write", "LEARN stage: append a best/failure/pattern entry to the knowledge file.",
                        {"report_ref": _S, "kind": {"type": "string", "enum": ["best", "failure", "pattern"]}},
                        ["report_ref", "kind"])

ALL_TOOLS = [RETURN_SUBAGENT_RESULT, WRITE_ARTIFACT, PREFLIGHT_RUN, ENV_PROBE_RUN, ENV_PROBE_SWEEP, PROFILER_RUN,
             SUBMIT_RUN, OBSERVE_SNAPSHOT, OBSERVE_COMPARE_LOSS, CONSTRAINT_CHECK, CONSTRAINT_CHECK_ENV,
             CONSTRAINT_ESTIMATE_MEM, KNOWLEDGE_WRITE]

_P = [WRITE_ARTIFACT, RETURN_SUBAGENT_RESULT]
STAGE_TOOL_MAP: dict[Stage, list[dict]] = {
    Stage.PREFLIGHT: [PREFLIGHT_RUN, ENV_PROBE_RUN, *_P],
    Stage.PROJECTION: [PROFILER_RUN, CONSTRAINT_ESTIMATE_MEM, *_P],
    Stage.SMOKE: [SUBMIT_RUN, OBSERVE_SNAPSHOT, *_P],
    Stage.BASELINE: [SUBMIT_RUN, OBSERVE_SNAPSHOT, *_P],
    Stage.CORRECTNESS: [OBSERVE_COMPARE_LOSS, RETURN_SUBAGENT_RESULT],
    Stage.OBSERVE: [OBSERVE_SNAPSHOT, *_P],
    Stage.DIAGNOSE: list(_P),
    Stage.REPLAN: [CONSTRAINT_CHECK, CONSTRAINT_CHECK_ENV, CONSTRAINT_ESTIMATE_MEM, *_P],
    Stage.ENV_SWEEP: [ENV_PROBE_SWEEP, CONSTRAINT_CHECK_ENV, *_P],
    Stage.CORRECTNESS_LITE: [OBSERVE_COMPARE_LOSS, RETURN_SUBAGENT_RESULT],
    Stage.SETTLE: list(_P),
    Stage.LEARN: [KNOWLEDGE_WRITE, RETURN_SUBAGENT_RESULT],
}


def tools_for_stage(stage: Stage) -> list[dict]:
    return STAGE_TOOL_MAP.get(stage, [RETURN_SUBAGENT_RESULT])


# ---------------------------------------------------------------------------------------------------------
# environment flag catalog (NVIDIA equivalents of the reference's ROCm-flavoured examples, env/SKILL.md)
# ---------------------------------------------------------------------------------------------------------
ENV_CATALOG = {
    "NCCL_NVLS_ENABLE": {"values": ["0", "1"], "axis": "cluster_shared", "note": "in-switch reduction"},
    "NCCL_BUFFSIZE": {"values": ["4194304", "8388608", "16777216"], "axis": "weakly_local"},
    "NCCL_MIN_NCHANNELS": {"values": ["8", "16", "32"], "axis": "weakly_local"},
    "NCCL_ALGO": {"values": ["Ring", "Tree", "NVLS"], "axis": "weakly_local"},
    "NCCL_PROTO": {"values": ["Simple", "LL128"], "axis": "weakly_local"},
    "CUDA_DEVICE_MAX_CONNECTIONS": {"values": ["1", "8", "32"], "axis": "weakly_local"},
    "PYTORCH_CUDA_ALLOC_CONF": {"values": ["expandable_segments:True", "max_split_size_mb:512"],
                                "axis": "weakly_local"},
    "TORCH_NCCL_AVOID_RECORD_STREAMS": {"values": ["0", "1"], "axis": "weakly_local"},
}
ENV_MUTEX = [({"NCCL_ALGO": "NVLS"}, {"NCCL_NVLS_ENABLE": "0"}, "NCCL_ALGO=NVLS needs NCCL_NVLS_ENABLE=1")]
ENV_WARN = {"NCCL_P2P_DISABLE": "disabling P2P removes the NVLink path the fused kernels rely on",
            "CUDA_LAUNCH_BLOCKING": "serialises every launch; never leave on for a measured run"}


def check_env(env_diff: dict) -> dict:
    violations, warnings = [], []
    for a, b, msg in ENV_MUTEX:
        if all(env_diff.get(k) == v for k, v in a.items()) and all(env_diff.get(k) == v for k, v in b.items()):
            violations.append(msg)
    for k, v in env_diff.items():
        if k in ENV_WARN and str(v) not in ("0", ""):
            warnings.append(f"{k}: {ENV_WARN[k]}")
        cat = ENV_CATALOG.get(k)
        if cat and str(v) not in cat["values"]:
            warnings.append(f"{k}={v} is outside the catalogued values {cat['values']}")
    return {"valid": not violations, "violations": violations, "warnings": warnings}


# ---------------------------------------------------------------------------------------------------------
# handlers
# ---------------------------------------------------------------------------------------------------------
class ToolContext:
    """What the handlers need: the state store, a job runner and the run's base configuration."""

    def __init__(self, store, runner=None, preset: str = "simplemoe-tiny", base_overrides=(), world: int = 1,
                 knowledge_path: Path | None = None):
        self.store, self.runner, self.preset = store, runner, preset
        self.base_overrides, self.world = list(base_overrides), world
        self.knowledge_path = knowledge_path or (store.session_dir / "knowledge.md")
        self.snapshots: dict[str, dict] = {}

    def load_plan(self, ref: str) -> dict:
        return json.loads(self.store.read_artifact(ref))

    def plan_config(self, plan: dict):
        from ...config import Config
        ov, _ = policy.plan_to_overrides(plan)
        cfg = Config()
        from ...models.presets import PRESETS
        cfg.update(PRESETS[self.preset])
        for o in self.base_overrides + ov:
            k, v = o.split("=", 1)
            cfg.set(k, v)
        return cfg


def _clock_state() -> dict | None:
    """SM clock and throttle reasons of GPU 0 right now (read-only query; None when nvidia-smi is not there)."""
    import subprocess
    q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    try:
        out = subprocess.run(["nvidia-smi", "-i", "0", f"--query-gpu={q}", "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=10).stdout.strip().splitlines()[0]
        f = [x.strip() for x in out.split(",")]
        reasons = [n for n, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[2:])
                   if v.lower() == "active"]
        return {"sm_mhz": float(f[0]), "sm_max_mhz": float(f[1]), "reasons": reasons,
                "throttled": any(r != "sw_power_cap" for r in reasons)}
    except Exception:
        return None


def preflight(cluster_id: str) -> dict:
    """ClusterProfile (``skills/pilot/workflow/preflight.md:72-107``): compute peaks, HBM, intra-node bandwidth.
    Uses the driver-written measured peaks when present; measures a GEMM and a copy when a GPU is visible."""
    import torch
    prof: dict[str, Any] = {"cluster_id": cluster_id, "collected_at": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()),
                            "nodes": 1, "gpus_per_node": torch.cuda.device_count() if torch.cuda.is_available() else 0,
                            "status": "tentative", "inter_node": None}
    peaks = Path(__file__).resolve().parents[3] / "MEASURED_PEAKS.json"
    if peaks.exists():
        mp = json.loads(peaks.read_text())
        prof.update(gpu_name=mp.get("gpu_name"), hbm_gbs=mp.get("hbm_gbs"), peak_tflops_bf16=mp.get("bf16_tflops"),
                    peak_tflops_bf16_sustained=mp.get("bf16_tflops_sustained"), status="validated")
    if torch.cuda.is_available():
        dev = torch.device("cuda")
        props = torch.cuda.get_device_properties(dev)
        prof.update(gpu_name=props.name, hbm_capacity_gb=props.total_memory / 2**30, sm_count=props.multi_processor_count)
        a = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)
        b = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)
        for _ in range(3):
            a @ b
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            a @ b
        e1.record()
        torch.cuda.synchronize()
        prof["peak_tflops_bf16_now"] = 10 * 2 * 8192**3 / (e0.elapsed_time(e1) * 1e-3) / 1e12
        prof["clocks_after_gemm"] = _clock_state()
        src = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
        dst = torch.empty_like(src)
        dst.copy_(src)
        e0.record()
        for _ in range(5):
            dst.copy_(src)
        e1.record()
        torch.cuda.synchronize()
        prof["hbm_gbs_now"] = 5 * 2 * (1 << 30) / (e0.elapsed_time(e1) * 1e-3) / 1e9
        prof["status"] = "validated"
    prof["supported_dtypes"] = ["fp32", "bf16", "fp8"] if prof.get("gpus_per_node") else ["fp32", "bf16"]
    prof["nvlink_gbs_per_direction_nominal"] = 900
    prof["env_baseline"] = {"NCCL_NVLS_ENABLE": "1"}
    return prof


def handle_tool_call(tool_name: str, tool_input: dict[str, Any], ctx) -> Any:
    """Route one tool call.  ``ctx`` is a :class:`ToolContext` (a bare StateStore is accepted for the two
    protocol tools)."""
    store = getattr(ctx, "store", ctx)
    if tool_name == "write_artifact":
        art = store.write_artifact(tool_input["kind"], tool_input["name"], tool_input["content"])
        return {"ref": art.ref, "size_bytes": art.size_bytes}
    if tool_name == "preflight_run":
        prof = preflight(tool_input["cluster_id"])
        art = store.write_artifact("ClusterProfile", f"{tool_input['cluster_id']}.json", json.dumps(prof, indent=2))
        return {"cluster_profile_ref": art.ref, "status": prof["status"], "gpus": prof["gpus_per_node"]}
    if tool_name == "env_probe_run":
        cands = tool_input.get("candidate_envs") or {}
        verdict = {k: check_env({k: v}) for k, v in cands.items()}
        art = store.write_artifact("EnvBaseline", "env_baseline.json", json.dumps(
            {"accepted": {k: v for k, v in cands.items() if verdict[k]["valid"]}, "verdict": verdict}, indent=2))
        return {"env_baseline_ref": art.ref}
    if tool_name == "constraint_check_env":
        return check_env(tool_input["env_diff"])
    if tool_name == "constraint_check":
        plan = ctx.load_plan(tool_input["plan_ref"])
        problems = check_config(ctx.plan_config(plan), ctx.world)
        return {"valid": not any(p["severity"] == "error" for p in problems),
                "violations": [p for p in problems if p["severity"] == "error"],
                "warnings": [p for p in problems if p["severity"] != "error"]}
    if tool_name == "constraint_estimate_mem":
        plan = ctx.load_plan(tool_input["plan_ref"])
        est = estimate_memory(ctx.plan_config(plan), ctx.world)
        return {"mem_gb": est["total_bytes"] / 2**30, "fits": est["fits"], "fraction_of_hbm": est["fraction"],
                "breakdown_gb": {k: est[k] / 2**30 for k in ("state_bytes", "transient_bytes", "activation_bytes",
                                                              "logits_bytes")}}
    if tool_name == "submit_run":
        plan = ctx.load_plan(tool_input["plan_ref"])
        job_id = ctx.runner.submit(plan, int(tool_input.get("max_steps") or 50),
                                   extra_overrides=list(tool_input.get("overrides") or []))
        return {"job_id": job_id}
    if tool_name == "observe_snapshot":
        job_id = tool_input["job_id"]
        snap = ctx.snapshots.get(job_id) or ctx.runner.wait(job_id)
        ctx.snapshots[job_id] = snap
        art = store.write_artifact("Snapshot", f"{job_id}.json", json.dumps(snap, indent=2))
        m = snap.get("metrics", {})
        return {"snapshot_ref": art.ref, "status": snap["status"], "tps": m.get("tps"),
                "step_time_ms": m.get("step_time_ms"), "comm_ratio": m.get("comm_ratio"),
                "bubble_ratio": m.get("bubble_ratio"), "mem_peak_gb": m.get("mem_peak_gb"),
                "completed_steps": snap.get("completed_steps")}
    if tool_name == "observe_compare_loss":
        snap = ctx.snapshots.get(tool_input["job_id"]) or ctx.runner.snapshot(tool_input["job_id"])
        ref = json.loads(store.read_artifact(tool_input["reference_curve_ref"]))
        ref_curve = ref["loss"]["curve"] if "loss" in ref else ref["curve"]
        return policy.compare_loss(snap["loss"]["curve"], ref_curve, lite=bool(tool_input.get("lite", False)))
    if tool_name == "env_probe_sweep":
        plan = ctx.load_plan(tool_input["base_plan_ref"])
        steps = min(int(tool_input.get("max_steps", 50)), 50)
        results = []
        combos = list(tool_input["candidate_envs"].items())[:8]          # caps: 5 flags / 8 combos / 50 steps
        for flag, value in combos:
            if not check_env({flag: value})["valid"]:
                continue
            q = json.loads(json.dumps(plan))
            q["id"] = f"{plan['id']}_env_{flag}"
            q.setdefault("env", {}).setdefault("diff", {})[flag] = value
            snap = ctx.runner.wait(ctx.runner.submit(q, steps, mode="envsweep"))
            results.append({"flag": flag, "value": value, "tps": snap.get("metrics", {}).get("tps"),
                            "status": snap["status"]})
        ok = [r for r in results if r["status"] == "ok" and r["tps"]]
        best = max(ok, key=lambda r: r["tps"]) if ok else None
        return {"best_env_diff": {best["flag"]: best["value"]} if best else {}, "results": results}
    if tool_name == "profiler_run":
        from ..projection import profile_micro_configs
        res = profile_micro_configs(ctx, tool_input.get("configs") or {})
        art = store.write_artifact("ProfilingResult", "projection.json", json.dumps(res, indent=2))
        return {"profiling_result_ref": art.ref, "fit": res.get("fit")}
    if tool_name == "knowledge_write":
        return write_knowledge(ctx.knowledge_path, store.read_artifact(tool_input["report_ref"]), tool_input["kind"])
    raise NotImplementedError(f"no handler for tool: {tool_name}")


def write_knowledge(path: Path, report_text: str, kind: str) -> dict:
    """Append an entry ``scope / evidence / rule / confidence / reproductions``; an entry whose rule already
    exists gets its reproduction count bumped and its confidence promoted (1 -> low, 2 -> medium, 3+ -> high)
    (``skills/pilot/knowledge/SKILL.md:14-125``)."""
    try:
        rep = json.loads(report_text)
    except json.JSONDecodeError:
        rep = {"rule": report_text.strip()[:300]}
    rule = rep.get("rule") or rep.get("headline") or "unspecified"
    path.parent.mkdir(parents=True, exist_ok=True)
    entries = []
    if path.exists():
        for block in path.read_text().split("\n## ")[1:]:
            lines = block.splitlines()
            e = {"title": lines[0]}
            for ln in lines[1:]:
                if ln.startswith("- ") and ":" in ln:
                    k, v = ln[2:].split(":", 1)
                    e[k.strip()] = v.strip()
            entries.append(e)
    for e in entries:
        if e.get("rule") == rule and e.get("kind") == kind:
            n = int(e.get("reproductions", "1")) + 1
            e["reproductions"] = str(n)
            e["confidence"] = "high" if n >= 3 else "medium"
            break
    else:
        entries.append({"title": f"{kind}: {rule[:60]}", "kind": kind, "scope": str(rep.get("scope", "single-node B200")),
                        "evidence": str(rep.get("evidence", rep.get("key_metrics", "")))[:300], "rule": rule,
                        "confidence": "low", "reproductions": "1"})
    text = "# Pilot knowledge\n"
    for e in entries:
        text += f"\n## {e['title']}\n" + "".join(f"- {k}: {e[k]}\n" for k in ("kind", "scope", "evidence", "rule",
                                                                              "confidence", "reproductions") if k in e)
    path.write_text(text)
    return {"written_paths": [str(path)], "entries": len(entries)}
