"""Job runner behind the tuner's ``submit_run`` / ``observe_snapshot`` tools.

``submit`` launches ``python -m system_lab_b200.train`` (under ``torch.distributed.run`` when the plan
needs more than one rank) as a child process with the plan's overrides and environment diff, asks it to
write its Snapshot when it finishes, and records the job under ``<session>/jobs/<job_id>/``.  ``wait``
polls the child: a job that prints nothing for ``hang_timeout_s`` (default 300 s, the reference's
single-node value, ``skills/pilot/workflow/execute.md:89-101``) or exceeds its wall-clock limit is stopped
by killing exactly the process group that was started, and the failure is classified
(``policy.classify_failure``) — the host-side half of failure detection; the device-side half is the
bounded waits in the kernels.
"""
from __future__ import annotations

import json
import os
import signal
import subprocess
import sys
import time
from pathlib import Path

from . import policy


class JobRunner:
    def __init__(self, jobs_dir: Path, preset: str, base_overrides=(), nproc: int = 1, device: str = "auto"):
        self.jobs_dir = Path(jobs_dir)
        self.preset, self.base_overrides, self.nproc, self.device = preset, list(base_overrides), nproc, device
        self._n = 0
        self.procs: dict[str, subprocess.Popen] = {}

    def submit(self, plan: dict, max_steps: int, *, mode: str = "challenger", timeout_s: float = 1800.0,
               extra_overrides=()) -> str:
        self._n += 1
        job_id = f"job_{self._n:04d}_{plan.get('id', 'plan')}"
        d = self.jobs_dir / job_id
        d.mkdir(parents=True, exist_ok=True)
        ov, env_diff = policy.plan_to_overrides(plan)
        world = plan["parallelism"]["dp"] * plan["parallelism"]["pp"] * plan["parallelism"].get("cp", 1)
        nproc = min(world, self.nproc) if self.nproc > 1 else 1
        ov = self.base_overrides + ov + list(extra_overrides) + [
            f"train_iters={max_steps}", f"snapshot_path={d / 'snapshot.json'}", f"device={self.device}", "log_interval=1"]
        repo_root = str(Path(__file__).resolve().parents[2])
        if nproc > 1:
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
                   "--master-addr", "127.0.0.1", "--master-port", str(29600 + self._n % 200),
                   "-m", "system_lab_b200.train", "--preset", self.preset, *ov]
        else:
            cmd = [sys.executable, "-m", "system_lab_b200.train", "--preset", self.preset, *ov]
        env = dict(os.environ, PYTHONPATH=repo_root + os.pathsep + os.environ.get("PYTHONPATH", ""), **env_diff)
        (d / "plan.json").write_text(json.dumps(plan, indent=2))
        (d / "cmd.json").write_text(json.dumps({"cmd": cmd, "env_diff": env_diff, "mode": mode,
                                                "timeout_s": timeout_s, "submitted_at": time.time()}))
        out = open(d / "stdout.log", "w")
        self.procs[job_id] = subprocess.Popen(cmd, stdout=out, stderr=subprocess.STDOUT, env=env, cwd=repo_root,
                                              start_new_session=True)
        return job_id

    def _kill(self, proc: subprocess.Popen) -> None:
        try:
            os.killpg(proc.pid, signal.SIGTERM)      # the group this runner created, nothing else
            proc.wait(timeout=10)
        except (ProcessLookupError, subprocess.TimeoutExpired):
            try:
                os.killpg(proc.pid, signal.SIGKILL)
            except ProcessLookupError:
                pass

    def wait(self, job_id: str, *, hang_timeout_s: float = policy.HANG_TIMEOUT_S, poll_s: float = 0.5) -> dict:
        """Block until the job ends (or is stopped) and return its Snapshot."""
        d = self.jobs_dir / job_id
        meta = json.loads((d / "cmd.json").read_text())
        proc = self.procs[job_id]
        log_path = d / "stdout.log"
        t0 = last_progress = time.time()
        last_size = 0
        stopped = None
        while proc.poll() is None:
            time.sleep(poll_s)
            size = log_path.stat().st_size if log_path.exists() else 0
            now = time.time()
            if size != last_size:
                last_size, last_progress = size, now
            if now - last_progress > hang_timeout_s:
                stopped = "hang"
                self._kill(proc)
                break
            if now - t0 > meta["timeout_s"]:
                stopped = "timeout"
                self._kill(proc)
                break
        rc = proc.returncode if proc.returncode is not None else -9
        return self.snapshot(job_id, exit_code=rc, stopped=stopped, wall_s=time.time() - t0)

    def snapshot(self, job_id: str, *, exit_code: int = 0, stopped: str | None = None, wall_s: float = 0.0) -> dict:
        d = self.jobs_dir / job_id
        plan = json.loads((d / "plan.json").read_text())
        snap_path = d / "snapshot.json"
        tail = ""
        if (d / "stdout.log").exists():
            tail = (d / "stdout.log").read_text(errors="replace")[-4000:]
        if snap_path.exists() and exit_code == 0:
            snap = json.loads(snap_path.read_text())
            snap.update(job_id=job_id, plan_id=plan.get("id", ""), exit_code=0, status="ok")
        else:
            kind = policy.classify_failure(exit_code, tail, timed_out=stopped == "timeout")
            status = {"OOM": "oom", "HANG": "hung", "TIMEOUT": "hung"}.get(kind, "failed")
            if stopped == "hang":
                kind, status = "HANG", "hung"
            snap = {"job_id": job_id, "plan_id": plan.get("id", ""), "status": status, "exit_code": exit_code,
                    "failure_kind": kind, "early_stop_reason": "hang_5min" if status == "hung" else None,
                    "completed_steps": tail.count("iteration "), "wall_time_s": wall_s,
                    "confidence_in_metrics": "low",
                    "metrics": {"tps": None, "mem_peak_gb": None, "has_nan": kind == "NUMERICAL"},
                    "loss": {"curve": []}, "resolved_env": {}, "log_tail": tail[-1500:]}
        snap["artifacts"] = {"stdout": str(d / "stdout.log"), "stderr": None, "trace": None}
        (d / "snapshot_final.json").write_text(json.dumps(snap, indent=2))
        return snap
