"""Orchestrator: the long-lived, deliberately thin agent that walks the tuning state machine.

Invariants kept from the reference (``pilot/agent/orchestrator.py:9-23``):

I1  every decision is made from the trimmed state alone — no conversation history is carried;
I2  the orchestrator has no business tools, only spawn / checkpoint / trim / handoff / stop;
I3  the state layer (files) is the only channel between iterations and between workers.

One ``step()`` = decide → apply → checkpoint → trim.  Decisions come from the LLM (exactly one tool call is
required, ``tool_choice=any``) or, for ``--dry-run`` and ``--backend rules``, from the deterministic stage
scheduler below, which also implements the on-fail edges and the anti-loop guard of the state machine
(``skills/pilot/workflow/state_machine.md:61-99``): a failed stage is retried once, the same failure kind three
times aborts, budgets are checked after every step.
"""
from __future__ import annotations

import json
import logging
from typing import Any

from .config import OrchestratorConfig
from .orchestrator_tools import ORCHESTRATOR_TOOLS
from .schemas import SpawnRequest, Stage, SubagentResult, OrchestratorState
from .skills import SkillLoader
from .state import StateStore
from .subagent import StageWorker
from .worker_tools import ToolContext

log = logging.getLogger(__name__)

MAX_SAME_FAILURE = 3

# skill globs per stage (mirrors prompts/orchestrator_base.md)
SKILL_SCOPE = {
    Stage.PREFLIGHT: ["workflow/preflight.md", "env/*", "profiling/*"],
    Stage.PROJECTION: ["workflow/projection.md", "execution-model/*", "constraints/*"],
    Stage.SMOKE: ["workflow/smoke.md", "workflow/execute.md"],
    Stage.BASELINE: ["workflow/baseline.md", "workflow/execute.md"],
    Stage.CORRECTNESS: ["workflow/correctness.md"],
    Stage.OBSERVE: ["workflow/observe.md"],
    Stage.DIAGNOSE: ["workflow/diagnose.md", "execution-model/*", "optimization/SKILL.md"],
    Stage.REPLAN: ["workflow/replan.md", "workflow/plan*.md", "workflow/axis_taxonomy.md", "optimization/*/SKILL.md",
                   "constraints/*"],
    Stage.EXECUTE: ["workflow/execute.md", "workflow/execution_strategy.md"],
    Stage.CORRECTNESS_LITE: ["workflow/correctness.md"],
    Stage.ENV_SWEEP: ["workflow/envsweep.md", "env/*", "constraints/env.md"],
    Stage.SETTLE: ["workflow/settle.md", "workflow/plan_graph.md"],
    Stage.LEARN: ["workflow/learn.md", "knowledge/*"],
}


class OrchestratorError(RuntimeError):
    pass


class Orchestrator:
    def __init__(self, cfg: OrchestratorConfig, client: Any | None = None, tools: ToolContext | None = None):
        cfg.ensure_dirs()
        self.cfg, self.client = cfg, client
        self.store = StateStore(cfg.session_dir)
        self.skills = SkillLoader(cfg.skills_dir)
        self.tools = tools or ToolContext(self.store)
        self.worker = StageWorker(cfg, client, self.skills, self.store, self.tools)
        self.llm = not cfg.dry_run and cfg.backend == "llm"
        if self.llm and client is None:
            raise OrchestratorError("an Anthropic client is required unless --dry-run or --backend rules is used")
        self.system_prompt = self._build_system_prompt()
        self.handed_off = False

    # ---------------------------------------------------------------------------------------- main loop
    def run(self) -> OrchestratorState:
        state = self.store.resume() or self.store.initial(self.cfg.session_id, self.cfg.budget_total)
        log.info("orchestrator start: session=%s stage=%s round=%d", state.session_id, state.current_stage.value,
                 state.round_id)
        while not state.is_terminal():
            state = self.step(state)
            if state.is_terminal():
                break
            if self._should_handoff(state):
                self.store.handoff(state, "context_pressure_auto")
                self.handed_off = True
                return state
            if state.budget_remaining().any_negative():
                log.info("budget exhausted -> REPORT")
                state.current_stage, state.stop_reason = Stage.REPORT, "BUDGET_EXCEEDED"
                self.store.checkpoint(state)
        log.info("orchestrator terminal: %s (%s)", state.current_stage.value, state.stop_reason)
        if not self.cfg.dry_run and self.store.latest_artifact("TuningReport") is None:
            from ..report import write_report
            try:
                log.info("report: %s", write_report(self.store, state))
            except Exception as e:                   # a report must never turn a finished session into a crash
                log.warning("could not write the tuning report: %s", e)
        return state

    def step(self, state: OrchestratorState) -> OrchestratorState:
        action = self._decide(state)
        state = self._apply(state, action)
        self.store.checkpoint(state)
        return self.store.trim(state)

    # ---------------------------------------------------------------------------------------- decide
    def _decide(self, state: OrchestratorState) -> dict:
        if not self.llm:
            return self._scheduled_action(state)
        user = json.dumps({"state": self.store.trim(state).model_dump(mode="json"),
                           "budget_remaining": state.budget_remaining().model_dump(),
                           "instruction": "Choose exactly one tool call."})
        resp = self.client.messages.create(model=self.cfg.orchestrator_model,
                                           max_tokens=self.cfg.orchestrator_response_tokens,
                                           system=self.system_prompt, tools=ORCHESTRATOR_TOOLS,
                                           tool_choice={"type": "any"},
                                           messages=[{"role": "user", "content": user}])
        state.budget_used.total_tokens += getattr(resp.usage, "input_tokens", 0) + getattr(resp.usage, "output_tokens", 0)
        uses = [b for b in resp.content if getattr(b, "type", None) == "tool_use"]
        if len(uses) != 1:
            raise OrchestratorError(f"expected exactly one tool call, got {len(uses)}")
        return {"name": uses[0].name, "input": dict(uses[0].input)}

    def _scheduled_action(self, state: OrchestratorState) -> dict:
        """Deterministic scheduler: spawn the worker for the current stage; apply the failure edges."""
        fails = [r for r in state.reentry_log if r.get("stage") == state.current_stage.value]
        if fails:
            kind = fails[-1].get("kind")
            same = state.failure_counts.get(kind, 0)
            if same >= MAX_SAME_FAILURE or kind in ("NUMERICAL",):
                return {"name": "orchestrator_stop", "input": {"reason": "ABORT", "summary": f"{kind} x{same}"}}
        if state.current_stage == Stage.OBSERVE and state.budget_total.rounds and \
                state.budget_used.rounds >= state.budget_total.rounds:
            return {"name": "orchestrator_stop", "input": {"reason": "BUDGET_EXCEEDED", "summary": "round budget used"}}
        return {"name": "subagent_spawn", "input": {
            "stage": state.current_stage.value, "skill_scope": SKILL_SCOPE.get(state.current_stage, []),
            "input_refs": {"cluster_profile": state.cluster_profile_ref, "plan_graph": state.plan_graph_ref,
                           "champion": state.champion_id, "round": state.round_id},
            "reason": "scheduled"}}

    # ---------------------------------------------------------------------------------------- apply
    def _apply(self, state: OrchestratorState, action: dict) -> OrchestratorState:
        name, arg = action["name"], action.get("input", {})
        if name == "subagent_spawn":
            req = SpawnRequest(stage=Stage(arg["stage"]), input_refs=arg.get("input_refs") or {},
                               skill_scope=arg.get("skill_scope") or [], max_tokens=int(arg.get("max_tokens", 30_000)),
                               parent_session=state.session_id)
            result = self.worker.run(req)
            return self._fold(state, result)
        if name == "state_checkpoint":
            self.store.checkpoint(state)
            return state
        if name == "state_trim":
            return self.store.trim(state)
        if name == "state_handoff":
            self.store.handoff(state, arg.get("reason", "requested"))
            self.handed_off = True
            state.current_stage, state.stop_reason = Stage.REPORT, "HANDOFF"
            return state
        if name == "orchestrator_stop":
            reason = arg.get("reason", "ABORT")
            state.stop_reason = reason
            state.current_stage = Stage.ABORT if reason == "ABORT" else Stage.REPORT
            state.last_decision_summary = arg.get("summary", reason)
            return state
        raise OrchestratorError(f"unknown orchestrator action {name!r}")

    def _fold(self, state: OrchestratorState, result: SubagentResult) -> OrchestratorState:
        if result.status == "success":
            return self.store.apply_result(state, result)
        # failure: budget is still charged, the stage stays (retry) and the failure is logged for the guard
        kind = result.failure.kind if result.failure else "UNKNOWN"
        state.failure_counts[kind] = state.failure_counts.get(kind, 0) + 1
        state.reentry_log.append({"stage": result.stage.value, "kind": kind, "round": state.round_id,
                                  "message": (result.failure.message if result.failure else "")[:200]})
        state.budget_used.total_tokens += int(result.cost.get("tokens_used", 0))
        state.budget_used.wallclock_h += float(result.cost.get("wallclock_s", 0.0)) / 3600.0
        state.budget_used.gpu_h += float(result.cost.get("gpu_h", 0.0))
        state.last_decision_summary = str(result.summary.get("headline", kind))
        state.stage_history.append({"round": state.round_id, "stage": result.stage.value, "status": result.status,
                                    "headline": state.last_decision_summary})
        if kind == "CONSTRAINT_VIOLATION" and result.stage in (Stage.EXECUTE, Stage.SMOKE):
            state.current_stage = Stage.REPLAN if result.stage == Stage.EXECUTE else Stage.PROJECTION
        elif kind == "OOM" and result.stage in (Stage.EXECUTE, Stage.BASELINE, Stage.SMOKE):
            state.current_stage = Stage.REPLAN if state.champion_id else Stage.PROJECTION
        return state

    # ---------------------------------------------------------------------------------------- guards
    def _should_handoff(self, state: OrchestratorState) -> bool:
        if not self.llm:
            return False
        tok = state.budget_total.total_tokens
        if tok and state.budget_used.total_tokens > self.cfg.handoff_token_ratio * tok:
            return True
        return state.round_id > 0 and state.round_id % self.cfg.max_rounds_before_handoff == 0 \
            and state.current_stage == Stage.OBSERVE

    def _build_system_prompt(self) -> str:
        base = (self.cfg.skills_dir.parent / "agent" / "prompts" / "orchestrator_base.md")
        here = __import__("pathlib").Path(__file__).parent / "prompts" / "orchestrator_base.md"
        text = (base if base.exists() else here).read_text()
        return "\n\n".join([text, "# State machine", self.skills.read("workflow/state_machine.md"),
                            "# Orchestration", self.skills.read("workflow/orchestration.md")])
