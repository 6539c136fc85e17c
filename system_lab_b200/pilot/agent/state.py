"""Filesystem state layer: the only channel between orchestrator iterations and between workers.

Layout under ``<state-dir>/<session>/``::

    checkpoints/s{seq:05d}_r{round:03d}_{STAGE}_{UTC}.json     one per orchestrator step
    handoffs/{UTC}_{reason}.json                               full state for a fresh orchestrator
    artifacts/{UTC}_{kind}_{name}                              heavy payloads written by workers
    jobs/<job_id>/                                             training runs launched by submit_run

Same operations as the reference's ``StateStore`` (``pilot/agent/state.py:42-160``).  File names start
with a zero-padded sequence number: the reference names files by second-resolution timestamp, so two
checkpoints of the same second sort by stage *name* and resume can pick the wrong one.
"""
from __future__ import annotations

import json
import logging
from pathlib import Path

from .schemas import Artifact, Budget, OrchestratorState, Stage, SubagentResult, utcnow

log = logging.getLogger(__name__)

KEEP_HISTORY = 3
KEEP_REENTRY = 1


def _ts() -> str:
    return utcnow().strftime("%Y%m%dT%H%M%SZ")


class StateStore:
    def __init__(self, session_dir: Path):
        self.session_dir = Path(session_dir)
        self.ckpt_dir = self.session_dir / "checkpoints"
        self.handoff_dir = self.session_dir / "handoffs"
        self.artifact_dir = self.session_dir / "artifacts"
        self.jobs_dir = self.session_dir / "jobs"
        for d in (self.ckpt_dir, self.handoff_dir, self.artifact_dir, self.jobs_dir):
            d.mkdir(parents=True, exist_ok=True)
        self._art_seq = 0

    def initial(self, session_id: str, budget_total: Budget) -> OrchestratorState:
        return OrchestratorState(session_id=session_id, current_stage=Stage.PREFLIGHT, budget_total=budget_total)

    def resume(self) -> OrchestratorState | None:
        files = sorted(self.ckpt_dir.glob("s*.json"))
        if not files:
            return None
        return OrchestratorState.model_validate_json(files[-1].read_text())

    def checkpoint(self, state: OrchestratorState) -> Path:
        state.seq += 1
        path = self.ckpt_dir / f"s{state.seq:05d}_r{state.round_id:03d}_{state.current_stage.name}_{_ts()}.json"
        path.write_text(state.model_dump_json(indent=2))
        return path

    def trim(self, state: OrchestratorState) -> OrchestratorState:
        """Keep pointers, budgets, the last few history lines; everything else stays on disk."""
        return state.model_copy(update={"stage_history": state.stage_history[-KEEP_HISTORY:],
                                        "reentry_log": state.reentry_log[-KEEP_REENTRY:]})

    def handoff(self, state: OrchestratorState, reason: str) -> Path:
        path = self.handoff_dir / f"{_ts()}_{reason}.json"
        path.write_text(json.dumps({"handoff_reason": reason, "handoff_at": utcnow().isoformat(),
                                    "state": state.model_dump(mode="json")}, indent=2))
        log.info("handoff written: %s", path)
        return path

    def resume_from_handoff(self, path: Path) -> OrchestratorState:
        return OrchestratorState.model_validate(json.loads(Path(path).read_text())["state"])

    def apply_result(self, state: OrchestratorState, result: SubagentResult) -> OrchestratorState:
        """Fold a worker result into the thin state: pointers by artifact kind, cost into the budget,
        SETTLE closes a round, the worker's suggested transition becomes the next stage."""
        state.last_decision_summary = str(result.summary.get("headline", ""))
        state.stage_history.append({"round": state.round_id, "stage": result.stage.value, "status": result.status,
                                    "headline": state.last_decision_summary, "at": utcnow().isoformat()})
        pointer = {"ClusterProfile": "cluster_profile_ref", "PlanGraph": "plan_graph_ref",
                   "TargetVector": "target_vector_ref", "Champion": "champion_id"}
        for art in result.artifacts:
            if art.kind in pointer:
                setattr(state, pointer[art.kind], art.ref)
        used = state.budget_used
        used.total_tokens += int(result.cost.get("tokens_used", 0))
        used.wallclock_h += float(result.cost.get("wallclock_s", 0.0)) / 3600.0
        used.gpu_h += float(result.cost.get("gpu_h", 0.0))
        if result.stage == Stage.SETTLE:
            state.round_id += 1
            used.rounds += 1
        if result.suggested_transition is not None:
            state.current_stage = result.suggested_transition.to
        return state

    def write_artifact(self, kind: str, name: str, content: str) -> Artifact:
        self._art_seq += 1
        path = self.artifact_dir / f"{_ts()}_{self._art_seq:04d}_{kind}_{name}"
        path.write_text(content)
        return Artifact(kind=kind, ref=str(path), size_bytes=path.stat().st_size)

    def read_artifact(self, ref: str) -> str:
        return Path(ref).read_text()

    def latest_artifact(self, kind: str) -> Path | None:
        files = sorted(self.artifact_dir.glob(f"*_{kind}_*"))
        return files[-1] if files else None
