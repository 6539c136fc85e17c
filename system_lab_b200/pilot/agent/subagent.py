"""Stage worker: a one-shot, isolated agent that runs a single stage and returns one SubagentResult.

Three back-ends:

* ``llm``     — the reference's loop (``pilot/agent/subagent.py:58-246``): system prompt = hard rules + the
  scoped skills, one JSON user message, at most ``MAX_TOOL_ROUNDTRIPS`` tool round-trips through the
  Messages API with the stage's tool set, ending in ``return_subagent_result``; protocol violations and
  budget overruns come back as ``status="failed"`` results instead of exceptions.
* ``rules``   — the same stages carried out by the deterministic policy (``pilot/policy.py``) calling the
  same tool handlers; no LLM, real jobs.  This is what makes the tuner usable and testable offline.
* dry run     — canned successes walking the default transition table, no jobs at all
  (``pilot/agent/subagent.py:251-313``).
"""
from __future__ import annotations

import json
import logging
import time
from typing import Any

from .. import policy
from .config import OrchestratorConfig
from .schemas import Artifact, SpawnRequest, Stage, SubagentFailure, SubagentResult, Transition
from .skills import SkillLoader
from .state import StateStore
from .worker_tools import ToolContext, handle_tool_call, tools_for_stage

log = logging.getLogger(__name__)

MAX_TOOL_ROUNDTRIPS = 12

_NEXT = {
    Stage.PREFLIGHT: Stage.PROJECTION, Stage.PROJECTION: Stage.SMOKE, Stage.SMOKE: Stage.BASELINE,
    Stage.BASELINE: Stage.CORRECTNESS, Stage.CORRECTNESS: Stage.OBSERVE, Stage.OBSERVE: Stage.DIAGNOSE,
    Stage.DIAGNOSE: Stage.REPLAN, Stage.REPLAN: Stage.EXECUTE, Stage.EXECUTE: Stage.CORRECTNESS_LITE,
    Stage.CORRECTNESS_LITE: Stage.SETTLE, Stage.ENV_SWEEP: Stage.SETTLE, Stage.SETTLE: Stage.OBSERVE,
    Stage.LEARN: Stage.REPORT,
}

HARD_RULES = """You are a stage worker of the Pilot training tuner. Rules:
1. Do exactly the stage you were given; never start another stage.
2. Use only the tools offered. Heavy data goes to write_artifact; your final answer is one call to
   return_subagent_result whose summary stays under ~200 tokens (headline + key_metrics).
3. Never invent measurements: every number in your summary comes from a tool result.
4. Suggest the next stage in suggested_transition; the orchestrator decides.
5. On a tool error, return status=failed with a failure kind instead of retrying blindly."""


class StageWorker:
    def __init__(self, cfg: OrchestratorConfig, client: Any, skills: SkillLoader, store: StateStore,
                 tools: ToolContext | None = None):
        self.cfg, self.client, self.skills, self.store = cfg, client, skills, store
        self.tools = tools or ToolContext(store)

    # ------------------------------------------------------------------------------------------ entry
    def run(self, req: SpawnRequest) -> SubagentResult:
        wid = f"{req.stage.name.lower()}_{int(time.time() * 1000) % 10**8}"
        t0 = time.time()
        try:
            if self.cfg.dry_run:
                res = self._dry_run(req, wid)
            elif self.cfg.backend == "rules":
                res = RuleWorker(self.cfg, self.store, self.tools).run(req, wid)
            else:
                res = self._run_llm(req, wid)
        except Exception as e:                      # a worker never takes the orchestrator down
            log.exception("worker %s crashed", wid)
            res = _failed(req.stage, wid, "TOOL_ERROR", f"{type(e).__name__}: {e}"[:300])
        res.cost.setdefault("wallclock_s", time.time() - t0)
        return res

    # ------------------------------------------------------------------------------------------ LLM loop
    def _system_prompt(self, req: SpawnRequest) -> str:
        scope = req.skill_scope or [f"workflow/{req.stage.name.lower()}.md"]
        return HARD_RULES + "\n\n# Skills in scope\n\n" + self.skills.read_scope(scope)

    def _run_llm(self, req: SpawnRequest, wid: str) -> SubagentResult:
        tools = tools_for_stage(req.stage)
        messages = [{"role": "user", "content": json.dumps(
            {"stage": req.stage.value, "input_refs": req.input_refs, "session": req.parent_session,
             "instruction": "Carry out this stage, then call return_subagent_result."})}]
        used = calls = 0
        for _ in range(MAX_TOOL_ROUNDTRIPS):
            resp = self.client.messages.create(model=self.cfg.worker_model, max_tokens=4096,
                                               system=self._system_prompt(req), tools=tools, messages=messages)
            used += getattr(resp.usage, "input_tokens", 0) + getattr(resp.usage, "output_tokens", 0)
            if used > req.max_tokens:
                return _failed(req.stage, wid, "TOKEN_BUDGET", f"worker used {used} tokens (cap {req.max_tokens})",
                               tokens=used, calls=calls)
            uses = [b for b in resp.content if getattr(b, "type", None) == "tool_use"]
            if not uses:
                return _failed(req.stage, wid, "UNKNOWN", "worker ended its turn without a tool call", tokens=used)
            final = next((b for b in uses if b.name == "return_subagent_result"), None)
            if final is not None:
                return self._from_return(req.stage, wid, final.input, used, calls)
            results = []
            for b in uses:
                calls += 1
                try:
                    out = handle_tool_call(b.name, b.input, self.tools)
                    results.append({"type": "tool_result", "tool_use_id": b.id, "content": json.dumps(out, default=str)})
                except Exception as e:
                    results.append({"type": "tool_result", "tool_use_id": b.id, "is_error": True,
                                    "content": f"{type(e).__name__}: {e}"})
            messages.append({"role": "assistant", "content": resp.content})
            messages.append({"role": "user", "content": results})
        return _failed(req.stage, wid, "TIMEOUT", f"no result after {MAX_TOOL_ROUNDTRIPS} tool round-trips",
                       tokens=used, calls=calls)

    def _from_return(self, stage: Stage, wid: str, payload: dict, tokens: int, calls: int) -> SubagentResult:
        try:
            tr = payload.get("suggested_transition")
            fl = payload.get("failure")
            return SubagentResult(
                stage=stage, worker_id=wid, status=payload["status"],
                artifacts=[Artifact(**a) for a in payload.get("artifacts", [])], summary=payload.get("summary", {}),
                suggested_transition=Transition(to=Stage(tr["to"]), reason=tr.get("reason", "")) if tr else None,
                failure=SubagentFailure(**fl) if fl else None, cost={"tokens_used": tokens, "tool_calls": calls})
        except Exception as e:
            return _failed(stage, wid, "UNKNOWN", f"malformed return_subagent_result: {e}"[:300], tokens=tokens)

    # ------------------------------------------------------------------------------------------ dry run
    def _dry_run(self, req: SpawnRequest, wid: str) -> SubagentResult:
        nxt = _NEXT.get(req.stage, Stage.REPORT)
        arts = []
        if req.stage == Stage.PREFLIGHT:
            arts.append(self.store.write_artifact("ClusterProfile", "dry.json", json.dumps({"cluster_id": "dry-run"})))
        if req.stage == Stage.REPLAN:
            arts.append(self.store.write_artifact("PlanGraph", "dry.json", "{}"))
        return SubagentResult(stage=req.stage, worker_id=wid, status="success", artifacts=arts,
                              summary={"headline": f"[dry-run] {req.stage.value} ok", "key_metrics": {}},
                              suggested_transition=Transition(to=nxt, reason="dry-run default edge"),
                              cost={"tokens_used": 200, "wallclock_s": 0.0, "gpu_h": 0.0, "tool_calls": 0})


def _failed(stage, wid, kind, msg, tokens=0, calls=0) -> SubagentResult:
    return SubagentResult(stage=stage, worker_id=wid, status="failed", summary={"headline": f"{stage.value} failed: {kind}"},
                          failure=SubagentFailure(kind=kind, message=msg), cost={"tokens_used": tokens, "tool_calls": calls})


# =====================================================================================================
# rule-based worker
# =====================================================================================================
class RuleWorker:
    """Runs each stage with the deterministic policy and the real tool handlers.  Session-wide working
    data (plan graph, champion snapshot, candidates) is kept in artifacts, as the skill pack prescribes."""

    SMOKE_STEPS, BASELINE_STEPS, CHALLENGER_STEPS = 6, 12, 12

    def __init__(self, cfg: OrchestratorConfig, store: StateStore, tools: ToolContext):
        self.cfg, self.store, self.tools = cfg, store, tools

    # -- small persistence helpers -----------------------------------------------------------------
    def _load(self, kind: str, default=None):
        p = self.store.latest_artifact(kind)
        return json.loads(p.read_text()) if p else default

    def _save(self, kind: str, name: str, obj) -> Artifact:
        return self.store.write_artifact(kind, name, json.dumps(obj, indent=2, default=str))

    def _graph(self) -> policy.PlanGraph:
        return policy.PlanGraph.from_dict(self._load("PlanGraph", {}))

    def _ok(self, stage, wid, headline, metrics=None, arts=(), to=None, gpu_h=0.0) -> SubagentResult:
        return SubagentResult(stage=stage, worker_id=wid, status="success", artifacts=list(arts),
                              summary={"headline": headline, "key_metrics": metrics or {}},
                              suggested_transition=Transition(to=to or _NEXT.get(stage, Stage.REPORT), reason="policy"),
                              cost={"tokens_used": 0, "gpu_h": gpu_h})

    def _run_plan(self, plan: dict, steps: int, mode: str, overrides=()) -> dict:
        ref = self._save("Plan", f"{plan['id']}.json", plan).ref
        job = handle_tool_call("submit_run", {"plan_ref": ref, "cluster_id": "local", "max_steps": steps,
                                              "overrides": list(overrides)}, self.tools)
        handle_tool_call("observe_snapshot", {"job_id": job["job_id"]}, self.tools)
        snap = self.tools.snapshots[job["job_id"]]
        snap["mode"] = mode
        return snap

    def _gpu_h(self, snap: dict) -> float:
        return (snap.get("wall_time_s") or 0.0) / 3600.0 * max(self.tools.world, 1)

    # -- stages ---------------------------------------------------------------------------------------
    def run(self, req: SpawnRequest, wid: str) -> SubagentResult:
        return getattr(self, "_" + req.stage.name.lower())(req, wid)

    def _preflight(self, req, wid):
        out = handle_tool_call("preflight_run", {"cluster_id": "local"}, self.tools)
        art = Artifact(kind="ClusterProfile", ref=out["cluster_profile_ref"])
        return self._ok(req.stage, wid, f"cluster profile {out['status']}, {out['gpus']} GPUs", out, [art])

    def _projection(self, req, wid):
        plan = policy.default_plan(self.tools.world)
        cfg = self.tools.plan_config(plan)
        plan["runtime"]["mbs"] = cfg.train.micro_batch_size
        plan["runtime"]["gbs"] = cfg.train.global_batch_size
        plan["parallelism"]["ep"] = min(cfg.parallel.expert_model_parallel_size, self.tools.world)
        plan["runtime"]["recompute"] = cfg.precision.recompute_granularity
        plan["comm"]["dispatcher"] = cfg.model.moe_token_dispatcher_type
        ref = self._save("Plan", "r0_p0.json", plan).ref
        mem = handle_tool_call("constraint_estimate_mem", {"plan_ref": ref}, self.tools)
        chk = handle_tool_call("constraint_check", {"plan_ref": ref}, self.tools)
        if not chk["valid"] or not mem["fits"]:
            return _failed(req.stage, wid, "CONSTRAINT_VIOLATION", json.dumps(chk["violations"])[:300])
        graph = policy.PlanGraph()
        graph.add(plan, "pending")
        arts = [self._save("PlanGraph", "graph.json", graph.to_dict()), Artifact(kind="TargetVector", ref=ref)]
        return self._ok(req.stage, wid, f"initial plan r0_p0, est {mem['mem_gb']:.1f} GB", {"mem_gb": mem["mem_gb"]}, arts)

    def _smoke(self, req, wid):
        graph = self._graph()
        plan = graph.nodes["r0_p0"]["plan"]
        # same parallel layout, everything else shrunk: at most 4 layers (a multiple of pp x vpp), micro-batch 1,
        # sequence at most 2048, full recompute
        cfg = self.tools.plan_config(plan)
        blocks = max(plan["parallelism"]["pp"] * plan["parallelism"].get("vpp", 1), 1)
        layers = max(min(cfg.model.num_layers, 4) // blocks * blocks, blocks)
        dp = plan["parallelism"]["dp"]
        shrink = [f"num_layers={layers}", f"first_k_dense={min(cfg.model.first_k_dense, layers - 1)}",
                  "micro_batch_size=1", f"global_batch_size={dp * max(plan['parallelism']['pp'], 1)}",
                  f"seq_length={min(cfg.model.seq_length, 2048)}", "recompute_granularity=full"]
        snap = self._run_plan(plan, self.SMOKE_STEPS, "smoke", shrink)
        if snap["status"] != "ok" or snap["metrics"].get("has_nan"):
            return _failed(req.stage, wid, snap.get("failure_kind", "UNKNOWN"), snap.get("log_tail", "")[-300:])
        return self._ok(req.stage, wid, f"smoke ok, {snap['completed_steps']} steps",
                        {"tps": snap["metrics"]["tps"]}, gpu_h=self._gpu_h(snap))

    def _baseline(self, req, wid):
        graph = self._graph()
        plan = graph.nodes["r0_p0"]["plan"]
        snap = self._run_plan(plan, self.BASELINE_STEPS, "baseline")
        if snap["status"] != "ok":
            return _failed(req.stage, wid, snap.get("failure_kind", "UNKNOWN"), snap.get("log_tail", "")[-300:])
        graph.nodes["r0_p0"].update(status="champion", tps=snap["metrics"]["tps"])
        graph.champion = "r0_p0"
        arts = [self._save("PlanGraph", "graph.json", graph.to_dict()), self._save("ChampionSnapshot", "r0_p0.json", snap),
                Artifact(kind="Champion", ref="r0_p0")]
        return self._ok(req.stage, wid, f"baseline tps {snap['metrics']['tps']:.0f}", {"tps": snap["metrics"]["tps"]},
                        arts, gpu_h=self._gpu_h(snap))

    def _correctness(self, req, wid):
        champ = self._load("ChampionSnapshot")
        curve = champ["loss"]["curve"]
        finite = all(l == l and abs(l) != float("inf") for _, l in curve)
        if not finite:
            return _failed(req.stage, wid, "NUMERICAL", "NaN/Inf in baseline loss curve")
        self._save("ReferenceCurve", "baseline.json", {"curve": curve})
        return self._ok(req.stage, wid, "reference curve = baseline (self-recompute fallback)", {"points": len(curve)})

    def _observe(self, req, wid):
        champ = self._load("ChampionSnapshot")
        return self._ok(req.stage, wid, f"champion {champ.get('plan_id')} tps {champ['metrics']['tps']:.0f}",
                        {k: champ["metrics"].get(k) for k in ("tps", "step_time_ms", "mem_peak_gb", "comm_ratio")})

    def _diagnose(self, req, wid):
        champ = self._load("ChampionSnapshot")
        rep = policy.diagnose(champ, expected_tps=(champ.get("metrics") or {}).get("expected_tps"))
        art = self._save("DiagnosisReport", "diag.json", rep)
        return self._ok(req.stage, wid, f"bottleneck {rep['bottleneck']} (conf {rep['confidence']:.1f})",
                        {"fired": rep["fired_rules"][:2]}, [art])

    def _replan(self, req, wid):
        graph, diag = self._graph(), self._load("DiagnosisReport")
        champion = graph.nodes[graph.champion]["plan"]
        state_round = int(req.input_refs.get("round", 0)) + 1

        def check(plan):
            ref = self._save("Plan", f"cand_{plan.get('id', 'x')}.json", plan).ref
            return handle_tool_call("constraint_check", {"plan_ref": ref}, self.tools)["violations"]

        def est(plan):
            ref = self._save("Plan", f"cand_{plan.get('id', 'x')}.json", plan).ref
            return handle_tool_call("constraint_estimate_mem", {"plan_ref": ref}, self.tools)["mem_gb"]

        cands = policy.replan(champion, diag, graph, check=check, estimate_mem=est, round_id=state_round,
                              top_k=2, explore=graph.rounds_without_gain >= 2)
        for c in cands:
            graph.add(c["plan"], "pending", axis=c["axis"])
        arts = [self._save("PlanGraph", "graph.json", graph.to_dict()),
                self._save("CandidatePool", f"r{state_round}.json", cands)]
        if not cands:
            return self._ok(req.stage, wid, "no legal candidate left", {}, arts, to=Stage.REPORT)
        return self._ok(req.stage, wid, f"{len(cands)} candidates: " + ", ".join(c["axis"] for c in cands),
                        {"top_priority": cands[0]["priority"]}, arts)

    def _execute(self, req, wid):
        graph = self._graph()
        pool = self._load("CandidatePool", [])
        results, gpu_h = [], 0.0
        for c in pool:
            snap = self._run_plan(c["plan"], self.CHALLENGER_STEPS, "challenger")
            gpu_h += self._gpu_h(snap)
            results.append({"plan_id": c["plan"]["id"], "status": snap["status"], "tps": snap["metrics"].get("tps"),
                            "curve": snap["loss"]["curve"], "failure_kind": snap.get("failure_kind")})
            self._save("Snapshot", f"{c['plan']['id']}.json", snap)
        art = self._save("ExecuteResults", "results.json", results)
        ok = [r for r in results if r["status"] == "ok"]
        return self._ok(req.stage, wid, f"{len(ok)}/{len(results)} challengers finished",
                        {"best_tps": max((r["tps"] or 0 for r in ok), default=None)}, [art], gpu_h=gpu_h)

    def _correctness_lite(self, req, wid):
        results = self._load("ExecuteResults", [])
        ref = self._load("ReferenceCurve", {"curve": []})
        for r in results:
            if r["status"] == "ok":
                cmp_ = policy.compare_loss(r["curve"], ref["curve"], tolerance=0.02, lite=True)
                r["correctness_ok"] = bool(cmp_["pass"])
                r["loss_delta_pct"] = cmp_["delta_pct"]
        art = self._save("ExecuteResults", "results_checked.json", results)
        bad = [r["plan_id"] for r in results if r["status"] == "ok" and not r.get("correctness_ok", True)]
        # a communication-bound champion with poor overlap also gets an environment sweep before settling
        to = Stage.ENV_SWEEP if self._load("DiagnosisReport", {}).get("env_suspect") else None
        return self._ok(req.stage, wid, f"loss gate: {len(bad)} rejected", {"rejected": bad[:4]}, [art], to=to)

    def _env_sweep(self, req, wid):
        """Only when the diagnosis flagged the environment (communication-bound with poor overlap): a handful of
        one-flag-at-a-time short runs on the champion; a winner joins this round's results as one more challenger."""
        diag = self._load("DiagnosisReport", {})
        if not diag.get("env_suspect"):
            return self._ok(req.stage, wid, "env sweep skipped (no env-suspect signal)", {})
        from .worker_tools import ENV_CATALOG
        graph = self._graph()
        champion = graph.nodes[graph.champion]["plan"]
        cur = champion.get("env", {}).get("diff", {})
        cands = {}
        for flag, spec in ENV_CATALOG.items():
            if spec["axis"] == "weakly_local" and flag.startswith("NCCL_") and len(cands) < 3:
                value = next((v for v in spec["values"] if cur.get(flag) != v), None)
                if value is not None:
                    cands[flag] = value
        ref = self._save("Plan", f"{champion['id']}_envbase.json", champion).ref
        out = handle_tool_call("env_probe_sweep", {"base_plan_ref": ref, "candidate_envs": cands,
                                                   "max_steps": self.CHALLENGER_STEPS}, self.tools)
        art = self._save("EnvSweepResult", "envsweep.json", out)
        best = max((r for r in out["results"] if r["status"] == "ok" and r["tps"]), key=lambda r: r["tps"], default=None)
        champ_tps = graph.nodes[graph.champion].get("tps") or 0.0
        arts = [art]
        if best and best["tps"] > champ_tps * (1 + policy.EPS_PROMOTE):
            q = json.loads(json.dumps(champion))
            q["id"] = f"{champion['id']}_env"
            q["parent"] = champion["id"]
            q.setdefault("env", {}).setdefault("diff", {})[best["flag"]] = best["value"]
            graph.add(q, "pending", axis=f"env.{best['flag']}")
            results = self._load("ExecuteResults", [])
            results.append({"plan_id": q["id"], "status": "ok", "tps": best["tps"], "curve": [], "failure_kind": None,
                            "correctness_ok": True})          # an environment flag does not change the arithmetic
            arts += [self._save("PlanGraph", "graph.json", graph.to_dict()),
                     self._save("ExecuteResults", "results_env.json", results)]
        return self._ok(req.stage, wid, f"env sweep: {len(out['results'])} probes, best {out['best_env_diff'] or 'none'}",
                        {"best": out["best_env_diff"]}, arts)

    def _settle(self, req, wid):
        graph, results = self._graph(), self._load("ExecuteResults", [])
        dec = policy.settle(graph, results)
        arts = [self._save("PlanGraph", "graph.json", graph.to_dict()), self._save("SettleDecision", "settle.json", dec)]
        if dec["promoted"]:
            snap_p = self.store.latest_artifact("Snapshot")
            for p in sorted(self.store.artifact_dir.glob("*_Snapshot_*")):
                if graph.champion in p.name:
                    snap_p = p
            arts.append(self._save("ChampionSnapshot", f"{graph.champion}.json", json.loads(snap_p.read_text())))
            arts.append(Artifact(kind="Champion", ref=graph.champion))
        to = Stage.REPORT if dec["stop"] else Stage.OBSERVE
        gain = dec["gain_vs_previous"]
        return self._ok(req.stage, wid, f"champion {graph.champion}" + (f" (+{100 * gain:.1f} %)" if gain else ""),
                        {"promoted": dec["promoted"], "stop": dec["stop"]}, arts, to=to)

    def _learn(self, req, wid):
        graph = self._graph()
        champ = graph.nodes.get(graph.champion or "", {})
        rep = {"rule": f"champion {graph.champion} via {champ.get('derived_axis')}", "scope": "single-node",
               "evidence": f"tps {champ.get('tps')}"}
        ref = self._save("Report", "learn.json", rep).ref
        out = handle_tool_call("knowledge_write", {"report_ref": ref, "kind": "best"}, self.tools)
        return self._ok(req.stage, wid, "knowledge updated", out, to=Stage.REPORT)
