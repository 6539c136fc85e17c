"""``python -m system_lab_b200.pilot.agent --session NAME [--dry-run | --backend rules]``

Same flags as the reference's ``python -m pilot.agent`` (``pilot/agent/__main__.py:15-30``): ``--session``
(required), ``--state-dir``, ``--skills-dir``, ``--gpu-h``, ``--max-rounds``, ``--wallclock-h``,
``--token-budget``, ``--orchestrator-model``, ``--worker-model``, ``--dry-run``, ``-v``; plus ``--backend rules``
(deterministic policy, real training jobs, no LLM), ``--preset``/``--override`` (what the jobs train) and
``--nproc``.  Without ``--dry-run``/``--backend rules`` an Anthropic client is created; exit code 2 if the
package or the API key is missing.
"""
from __future__ import annotations

import argparse
import logging
import os
import sys
from pathlib import Path

from .config import DEFAULT_ORCHESTRATOR_MODEL, DEFAULT_WORKER_MODEL, OrchestratorConfig
from .orchestrator import Orchestrator
from .schemas import Budget
from .worker_tools import ToolContext

_DEFAULT_SKILLS = Path(__file__).resolve().parent.parent / "skills"


def parse_args(argv=None) -> argparse.Namespace:
    ap = argparse.ArgumentParser("pilot-agent")
    ap.add_argument("--session", required=True)
    ap.add_argument("--state-dir", default="pilot/state", type=Path)
    ap.add_argument("--skills-dir", default=_DEFAULT_SKILLS, type=Path)
    ap.add_argument("--gpu-h", type=float, default=10.0)
    ap.add_argument("--max-rounds", type=int, default=5)
    ap.add_argument("--wallclock-h", type=float, default=24.0)
    ap.add_argument("--token-budget", type=int, default=400_000)
    ap.add_argument("--orchestrator-model", default=DEFAULT_ORCHESTRATOR_MODEL)
    ap.add_argument("--worker-model", default=DEFAULT_WORKER_MODEL)
    ap.add_argument("--dry-run", action="store_true", help="no LLM, no jobs: canned worker results")
    ap.add_argument("--backend", choices=["llm", "rules"], default="llm")
    ap.add_argument("--preset", default="simplemoe-tiny")
    ap.add_argument("--override", action="append", default=[], help="trainer key=value (repeatable)")
    ap.add_argument("--nproc", type=int, default=1)
    ap.add_argument("--device", default="auto")
    ap.add_argument("-v", "--verbose", action="count", default=0)
    return ap.parse_args(argv)


def main(argv=None) -> int:
    args = parse_args(argv)
    logging.basicConfig(level=logging.DEBUG if args.verbose else logging.INFO,
                        format="%(asctime)s %(levelname)-7s %(name)s :: %(message)s")
    cfg = OrchestratorConfig(
        session_id=args.session, session_dir=args.state_dir / args.session, skills_dir=args.skills_dir,
        budget_total=Budget(gpu_h=args.gpu_h, rounds=args.max_rounds, wallclock_h=args.wallclock_h,
                            total_tokens=args.token_budget),
        orchestrator_model=args.orchestrator_model, worker_model=args.worker_model, dry_run=args.dry_run,
        backend=args.backend, train_preset=args.preset, train_overrides=tuple(args.override), nproc=args.nproc)
    client = None
    if not cfg.dry_run and cfg.backend == "llm":
        try:
            from anthropic import Anthropic
        except ImportError:
            print("anthropic package missing; use --dry-run or --backend rules", file=sys.stderr)
            return 2
        if "ANTHROPIC_API_KEY" not in os.environ:
            print("ANTHROPIC_API_KEY not set; use --dry-run or --backend rules", file=sys.stderr)
            return 2
        client = Anthropic()
    cfg.ensure_dirs()
    from .state import StateStore
    from ..runner import JobRunner
    store = StateStore(cfg.session_dir)
    runner = JobRunner(store.jobs_dir, cfg.train_preset, cfg.train_overrides, cfg.nproc, args.device)
    tools = ToolContext(store, runner, cfg.train_preset, cfg.train_overrides, world=max(cfg.nproc, 1))
    orch = Orchestrator(cfg, client, tools)
    orch.store = store
    orch.worker.store = store
    state = orch.run()
    print(f"\n=== done ===\nfinal stage: {state.current_stage.value}\nrounds: {state.round_id}\n"
          f"tokens used: {state.budget_used.total_tokens}\nsummary: {state.last_decision_summary}\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
