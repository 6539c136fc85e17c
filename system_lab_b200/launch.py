"""``python -m system_lab_b200.launch --nproc N [--max-restarts R] [--shrink] -- <train arguments>``

A supervisor for one node: starts one training process per rank, watches them, and when a rank fails (non-zero
exit, a ``PeerFailure`` raised from the heartbeat watchdog, a crash) stops the remaining ranks, then starts the job
again from the newest complete checkpoint.  With ``--shrink`` a restart may use fewer ranks (half, while the
configuration stays legal): checkpoints are layout-independent, so the smaller job reshards on load.

The supervisor never touches a GPU.  Ranks are stopped between steps where possible: a healthy rank learns of the
failure from the heartbeat store (``trainer/watchdog.py``) and leaves before it launches its next step; the
supervisor then signals only the process groups it created itself (SIGTERM, SIGKILL after a grace period).

Fault plans (``fault_injection=...``) apply to the first attempt only: restarted ranks see ``SLAB_RESTART_COUNT > 0``
and ignore them, so an injected failure cannot repeat forever.

Reference: the reference describes recovery practice for large jobs (healthy-node pools, replace-node-keep-
topology, ``summary/training-1024g*:41-101``; hot replicas and < 30 s recovery in the MegaScale-MoE digest,
``moe/MegaScale_MoE_reading_notes.md:156-231``) and the tuner's failure kinds (``skills/pilot/constraints/
validation.md:28-147``) but ships no launcher, membership or restart code.
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import socket
import subprocess
import sys
import time
from pathlib import Path


def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _resolve(train_args: list[str]):
    """The job's configuration, resolved the way ``train.py`` resolves it (defaults < preset < YAML < overrides)."""
    from .config import Config
    preset, config, overrides = None, None, []
    it = iter(train_args)
    for a in it:
        if a == "--preset":
            preset = next(it)
        elif a == "--config":
            config = next(it)
        elif a == "--resume":
            next(it)
        elif not a.startswith("--"):
            overrides.append(a)
    return Config.load(config, overrides, preset)


def _save_dir(train_args: list[str]) -> str:
    """The checkpoint directory the job writes to (``checkpoint.save``, from any configuration layer), or ''."""
    from .config import ConfigError
    try:
        return _resolve(train_args).checkpoint.save
    except ConfigError:
        return ""


def newest_checkpoint(root: str) -> str:
    """Newest complete checkpoint under ``root`` (a ``step_*`` directory with its ``meta.json``), or ''."""
    if not root or not Path(root).is_dir():
        return ""
    done = [d for d in sorted(Path(root).glob("step_*")) if (d / "meta.json").exists()]
    return str(done[-1]) if done else ""


def _legal(train_args: list[str], world: int) -> bool:
    from .config import ConfigError
    try:
        _resolve(train_args).validate(world)
        return True
    except ConfigError:
        return False


class Supervisor:
    def __init__(self, nproc: int, train_args: list[str], *, max_restarts: int = 3, shrink: bool = False,
                 min_nproc: int = 1, grace_s: float = 10.0, poll_s: float = 0.2, log_dir: str = "",
                 python: str = sys.executable, bind_cores: bool = False):
        self.nproc, self.train_args = nproc, list(train_args)
        self.max_restarts, self.shrink, self.min_nproc = max_restarts, shrink, min_nproc
        self.grace_s, self.poll_s = grace_s, poll_s
        self.log_dir = Path(log_dir) if log_dir else None
        self.python = python
        # bind_cores: every rank gets its own contiguous slice of the host's cores (the data-loader and launch
        # threads of different ranks then do not migrate onto each other's cores; the reference's large-job notes
        # bind ranks to the NUMA node of their GPU, ``summary/training-1024g*:41-101``)
        self.bind_cores = bind_cores
        self.history: list[dict] = []

    # ---- one attempt -----------------------------------------------------------------------------------
    def _spawn(self, world: int, attempt: int, resume: str) -> list[subprocess.Popen]:
        port = _free_port()
        procs = []
        args = [a for a in self.train_args]
        if resume:
            args = ["--resume", resume] + args
        for rank in range(world):
            env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
                       MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), SLAB_RESTART_COUNT=str(attempt))
            if world > 1:
                env.setdefault("OMP_NUM_THREADS", str(max((os.cpu_count() or world) // world, 1)))
            out = subprocess.DEVNULL
            if self.log_dir is not None:
                self.log_dir.mkdir(parents=True, exist_ok=True)
                out = open(self.log_dir / f"attempt{attempt}_rank{rank}.log", "w")
            # a session of its own: stopping the rank signals this process group and nothing else
            procs.append(subprocess.Popen([self.python, "-m", "system_lab_b200.train"] + args, env=env, stdout=out,
                                          stderr=subprocess.STDOUT, start_new_session=True,
                                          preexec_fn=self._binder(rank, world)))
        return procs

    def _binder(self, rank: int, world: int):
        if not self.bind_cores or not hasattr(os, "sched_setaffinity"):
            return None
        cores = sorted(os.sched_getaffinity(0))
        per = len(cores) // world
        if per < 1:
            return None
        mine = set(cores[rank * per:(rank + 1) * per])
        return lambda: os.sched_setaffinity(0, mine)

    def _stop(self, procs: list[subprocess.Popen]) -> None:
        for sig, wait in ((signal.SIGTERM, self.grace_s), (signal.SIGKILL, 5.0)):
            alive = [p for p in procs if p.poll() is None]
            if not alive:
                return
            for p in alive:
                try:
                    os.killpg(p.pid, sig)
                except ProcessLookupError:
                    pass
            end = time.time() + wait
            while time.time() < end and any(p.poll() is None for p in alive):
                time.sleep(0.05)

    def _watch(self, procs: list[subprocess.Popen]) -> dict:
        """Wait until every rank has exited 0, or one has failed (then give the others the grace period to leave on
        their own, which they do once the heartbeat reports the failure, and stop whoever remains)."""
        while True:
            codes = [p.poll() for p in procs]
            failed = [(r, c) for r, c in enumerate(codes) if c not in (None, 0)]
            if failed:
                end = time.time() + self.grace_s
                while time.time() < end and any(p.poll() is None for p in procs):
                    time.sleep(self.poll_s)
                self._stop(procs)
                return {"ok": False, "first_failed_rank": failed[0][0], "exit_code": failed[0][1],
                        "exit_codes": [p.poll() for p in procs]}
            if all(c == 0 for c in codes):
                return {"ok": True, "exit_codes": codes}
            time.sleep(self.poll_s)

    # ---- the restart loop ---------------------------------------------------------------------------------
    def run(self) -> int:
        world, attempt = self.nproc, 0
        save = _save_dir(self.train_args)
        while True:
            resume = newest_checkpoint(save) if attempt > 0 else ""
            t0 = time.time()
            procs = self._spawn(world, attempt, resume)
            try:
                res = self._watch(procs)
            except BaseException:
                self._stop(procs)
                raise
            res.update(attempt=attempt, world=world, resumed_from=resume, wall_s=round(time.time() - t0, 2))
            self.history.append(res)
            print(json.dumps({"launch": res}), flush=True)
            if res["ok"]:
                return 0
            if attempt >= self.max_restarts:
                return 1
            attempt += 1
            if self.shrink and world // 2 >= self.min_nproc and _legal(self.train_args, world // 2):
                world //= 2


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    train_args = []
    if "--" in argv:
        i = argv.index("--")
        argv, train_args = argv[:i], argv[i + 1:]
    ap = argparse.ArgumentParser("system_lab_b200.launch")
    ap.add_argument("--nproc", type=int, default=1)
    ap.add_argument("--max-restarts", type=int, default=3)
    ap.add_argument("--shrink", action="store_true", help="a restart may halve the number of ranks")
    ap.add_argument("--min-nproc", type=int, default=1)
    ap.add_argument("--grace-s", type=float, default=10.0)
    ap.add_argument("--log-dir", default="")
    ap.add_argument("--bind-cores", action="store_true", help="give every rank its own slice of the host's cores")
    a = ap.parse_args(argv)
    sup = Supervisor(a.nproc, train_args, max_restarts=a.max_restarts, shrink=a.shrink, min_nproc=a.min_nproc,
                     grace_s=a.grace_s, log_dir=a.log_dir, bind_cores=a.bind_cores)
    return sup.run()


if __name__ == "__main__":
    sys.exit(main())
