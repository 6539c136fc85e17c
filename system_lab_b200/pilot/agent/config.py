"""Agent configuration (``pilot/agent/config.py:13-41`` of the reference): model slugs, context hygiene
thresholds, dry-run switch, session directories."""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

from .schemas import Budget

DEFAULT_ORCHESTRATOR_MODEL = "claude-opus-4-5-20250929"
DEFAULT_WORKER_MODEL = "claude-opus-4-5-20250929"


@dataclass
class OrchestratorConfig:
    session_id: str
    session_dir: Path
    skills_dir: Path
    budget_total: Budget
    orchestrator_model: str = DEFAULT_ORCHESTRATOR_MODEL
    worker_model: str = DEFAULT_WORKER_MODEL
    orchestrator_response_tokens: int = 2_048
    worker_max_tokens: int = 30_000
    handoff_token_ratio: float = 0.5         # hand off when tokens used exceed this share of the budget
    max_rounds_before_handoff: int = 15
    dry_run: bool = False                    # canned worker results, no LLM, no jobs
    backend: str = "llm"                     # llm | rules (deterministic policy drives real tools)
    train_preset: str = "simplemoe-tiny"     # what submit_run launches
    train_overrides: tuple = ()
    nproc: int = 1
    scratch_dir: Path | None = None

    def ensure_dirs(self) -> None:
        for sub in ("checkpoints", "handoffs", "artifacts", "jobs"):
            (self.session_dir / sub).mkdir(parents=True, exist_ok=True)
