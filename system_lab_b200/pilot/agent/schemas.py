"""Wire formats between orchestrator, stage workers and the state layer (pydantic models).

Behavioural parity with ``pilot/agent/schemas.py:20-182`` of the reference: the same 15 stage values, the
same split between delegated and inline stages, the same failure kinds, the 1200-character cap on a
worker's summary (details belong in artifacts)."""
from __future__ import annotations

import json
from datetime import datetime, timezone
from enum import Enum
from typing import Any, Literal

from pydantic import BaseModel, Field, field_validator

SUMMARY_CHAR_CAP = 1200


class Stage(str, Enum):
    PREFLIGHT = "PREFLIGHT"
    PROJECTION = "PROJECTION"
    SMOKE = "SMOKE"
    BASELINE = "BASELINE"
    CORRECTNESS = "CORRECTNESS"
    OBSERVE = "OPTIMIZE_LOOP.OBSERVE"
    DIAGNOSE = "OPTIMIZE_LOOP.DIAGNOSE"
    REPLAN = "OPTIMIZE_LOOP.REPLAN"
    EXECUTE = "OPTIMIZE_LOOP.EXECUTE"
    CORRECTNESS_LITE = "OPTIMIZE_LOOP.CORRECTNESS_LITE"
    ENV_SWEEP = "OPTIMIZE_LOOP.ENV_SWEEP"
    SETTLE = "OPTIMIZE_LOOP.SETTLE"
    REPORT = "REPORT"
    LEARN = "LEARN"
    ABORT = "ABORT"


SUBAGENT_STAGES = frozenset({Stage.PREFLIGHT, Stage.PROJECTION, Stage.OBSERVE, Stage.DIAGNOSE, Stage.REPLAN,
                             Stage.ENV_SWEEP, Stage.CORRECTNESS_LITE, Stage.SMOKE, Stage.CORRECTNESS, Stage.LEARN})
ORCHESTRATOR_INLINE_STAGES = frozenset({Stage.EXECUTE, Stage.SETTLE, Stage.BASELINE})
TERMINAL_STAGES = frozenset({Stage.REPORT, Stage.ABORT})

FailureKind = Literal["SKILL_MISSING", "TOOL_ERROR", "CONSTRAINT_VIOLATION", "TIMEOUT", "TOKEN_BUDGET", "OOM",
                      "HANG", "NUMERICAL", "UNKNOWN"]
StopReason = Literal["CONVERGED", "BUDGET_EXCEEDED", "ABORT", "STAGNATION"]


def utcnow() -> datetime:
    return datetime.now(timezone.utc)


class Budget(BaseModel):
    gpu_h: float = 0.0
    rounds: int = 0
    wallclock_h: float = 0.0
    total_tokens: int = 0

    def minus(self, other: "Budget") -> "Budget":
        return Budget(gpu_h=self.gpu_h - other.gpu_h, rounds=self.rounds - other.rounds,
                      wallclock_h=self.wallclock_h - other.wallclock_h,
                      total_tokens=self.total_tokens - other.total_tokens)

    def any_negative(self) -> bool:
        return min(self.gpu_h, self.rounds, self.wallclock_h, self.total_tokens) < 0


class OrchestratorState(BaseModel):
    """The thin state the orchestrator carries: pointers and one-line summaries, never payloads."""
    session_id: str
    current_stage: Stage
    round_id: int = 0
    seq: int = 0                                  # monotonic checkpoint sequence number
    champion_id: str | None = None
    cluster_profile_ref: str | None = None
    plan_graph_ref: str | None = None
    target_vector_ref: str | None = None
    budget_total: Budget
    budget_used: Budget = Field(default_factory=Budget)
    last_decision_summary: str = ""
    stop_reason: str | None = None
    stage_history: list[dict[str, Any]] = Field(default_factory=list)
    reentry_log: list[dict[str, Any]] = Field(default_factory=list)
    failure_counts: dict[str, int] = Field(default_factory=dict)   # per failure kind; survives trimming

    def budget_remaining(self) -> Budget:
        return self.budget_total.minus(self.budget_used)

    def is_terminal(self) -> bool:
        return self.current_stage in TERMINAL_STAGES


class Artifact(BaseModel):
    kind: str
    ref: str
    size_bytes: int = 0


class Transition(BaseModel):
    to: Stage
    reason: str = ""


class SubagentFailure(BaseModel):
    kind: FailureKind
    message: str = ""
    escalate_to_orchestrator: bool = False


class SubagentResult(BaseModel):
    stage: Stage
    worker_id: str
    status: Literal["success", "failed", "escalate"]
    artifacts: list[Artifact] = Field(default_factory=list)
    summary: dict[str, Any] = Field(default_factory=dict)
    suggested_transition: Transition | None = None
    cost: dict[str, Any] = Field(default_factory=dict)      # tokens_used, wallclock_s, gpu_h, tool_calls
    failure: SubagentFailure | None = None
    created_at: datetime = Field(default_factory=utcnow)

    @field_validator("summary")
    @classmethod
    def _cap(cls, v: dict[str, Any]) -> dict[str, Any]:
        n = len(json.dumps(v, ensure_ascii=False, default=str))
        if n > SUMMARY_CHAR_CAP:
            raise ValueError(f"summary is {n} chars; the cap is {SUMMARY_CHAR_CAP}. Put detail in artifacts "
                             "and keep the summary to a headline plus key metrics.")
        return v


class SpawnRequest(BaseModel):
    stage: Stage
    input_refs: dict[str, Any] = Field(default_factory=dict)
    skill_scope: list[str] = Field(default_factory=list)
    max_tokens: int = 30_000
    parent_session: str = ""
