"""Host-side failure detection and fault injection for the trainer.

Device side, every wait is bounded and ends in a status word (``ops/cuda.py: check_status`` -> ``DeviceHang``).
This module is the host side: ranks publish a heartbeat through the process group's store after every step, a
watchdog thread on each rank compares the peers' heartbeats with its own progress, and a rank that falls behind
for longer than ``hang_timeout_s`` (or stops publishing, or publishes an error) is reported *before the next
step is launched*, so no kernel or collective is in flight when the healthy ranks raise ``PeerFailure`` and
leave.  Nothing here touches a GPU.

Fault injection is host-only by construction: a rank can be delayed, made to raise, made to exit, made to
produce a NaN loss, or made to stop its heartbeat at a chosen step (``FaultPlan``, parsed from
``train.fault_injection``); tests use it with gloo ranks on CPU.

Reference: failure kinds and routing ``skills/pilot/constraints/validation.md:28-147``, hang rules
``skills/pilot/workflow/execute.md:89-101``; the reference ships no heartbeat, membership or injection code.
"""
from __future__ import annotations

import os
import threading
import time
from dataclasses import dataclass, field


class PeerFailure(RuntimeError):
    """Another rank hung, died or reported an error (failure kind HANG or CLUSTER)."""

    def __init__(self, kind: str, rank: int, detail: str):
        super().__init__(f"{kind}: rank {rank}: {detail}")
        self.kind, self.rank, self.detail = kind, rank, detail


class InjectedFault(RuntimeError):
    """Raised by ``FaultPlan`` on the rank and step the plan names."""


@dataclass
class FaultPlan:
    """``"delay:rank=1,step=3,seconds=5;raise:rank=0,step=4"`` -> actions keyed by (rank, step).

    kinds: ``delay`` (sleep ``seconds`` before the step), ``raise`` (raise ``InjectedFault``), ``exit`` (``os._exit``
    with ``code``, default 17: a rank that vanishes without saying anything), ``nan`` (the step reports a NaN loss),
    ``mute`` (stop publishing heartbeats from that step on, the rank itself keeps running)."""
    actions: list = field(default_factory=list)

    @staticmethod
    def parse(spec: str) -> "FaultPlan":
        plan = FaultPlan()
        for part in filter(None, (p.strip() for p in (spec or "").split(";"))):
            kind, _, rest = part.partition(":")
            kv = dict(x.split("=", 1) for x in rest.split(",") if "=" in x)
            if kind not in ("delay", "raise", "exit", "nan", "mute"):
                raise ValueError(f"unknown fault kind {kind!r}")
            plan.actions.append({"kind": kind, "rank": int(kv.get("rank", 0)), "step": int(kv.get("step", 1)),
                                 "seconds": float(kv.get("seconds", 0)), "code": int(kv.get("code", 17))})
        return plan

    def at(self, rank: int, step: int) -> list:
        return [a for a in self.actions if a["rank"] == rank and a["step"] == step]

    def before_step(self, rank: int, step: int) -> dict:
        """Apply the host-side actions for this rank and step; returns flags the trainer honours (``nan``, ``mute``)."""
        flags = {}
        for a in self.at(rank, step):
            if a["kind"] == "delay":
                time.sleep(a["seconds"])
            elif a["kind"] == "raise":
                raise InjectedFault(f"injected failure on rank {rank} at step {step}")
            elif a["kind"] == "exit":
                os._exit(a["code"])
            else:
                flags[a["kind"]] = True
        return flags


class Heartbeat:
    """Per-rank heartbeat over a c10d store plus a watchdog thread.

    Progress is counted in half steps: ``begin(step)`` publishes ``2*step - 1`` when the rank starts a step,
    ``beat(step)`` publishes ``2*step`` when it has finished one (``hb/<rank> = "<progress> <time> ok"``);
    ``fail(msg)`` publishes an error so the peers need not wait for the timeout.  A peer whose progress is behind
    this rank's and has not moved for ``timeout_s`` is hung: typically this rank sits in the step's first
    collective waiting for a peer that never started the step.  ``check()`` (called by the trainer before it
    launches a step) raises the ``PeerFailure`` the watchdog thread recorded."""

    def __init__(self, store, rank: int, world: int, timeout_s: float, poll_s: float = 0.25, prefix: str = "hb"):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s, self.poll_s, self.prefix = timeout_s, poll_s, prefix
        self.muted = False
        self._failure: PeerFailure | None = None
        self._stop = threading.Event()
        self._last_seen = {r: (0, time.time()) for r in range(world)}        # rank -> (step, local time first seen)
        self._my_step = 0
        self._thread = None

    def start(self) -> "Heartbeat":
        self.beat(0)
        if self.world > 1:
            self._thread = threading.Thread(target=self._watch, name="slab-heartbeat", daemon=True)
            self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.poll_s + 1)

    def _publish(self, progress: int) -> None:
        self._my_step = progress
        if not self.muted:
            self.store.set(f"{self.prefix}/{self.rank}", f"{progress} {time.time():.3f} ok")

    def begin(self, step: int) -> None:
        self._publish(2 * step - 1)

    def beat(self, step: int) -> None:
        self._publish(2 * step)

    def fail(self, message: str) -> None:
        try:
            self.store.set(f"{self.prefix}/{self.rank}", f"{self._my_step} {time.time():.3f} error {message[:200]}")
        except Exception:
            pass

    def check(self) -> None:
        if self._failure is not None:
            raise self._failure

    # ---- watchdog thread ---------------------------------------------------------------------------
    def _read(self, r: int):
        key = f"{self.prefix}/{r}"
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:
            return None

    def _watch(self) -> None:
        while not self._stop.is_set() and self._failure is None:
            now = time.time()
            for r in range(self.world):
                if r == self.rank:
                    continue
                val = self._read(r)
                if val is None:
                    step, state, msg = 0, "ok", ""
                else:
                    parts = val.split(" ", 3)
                    step, state, msg = int(parts[0]), parts[2], (parts[3] if len(parts) > 3 else "")
                if state == "error":
                    self._failure = PeerFailure("CLUSTER", r, f"reported: {msg}")
                    return
                seen_step, since = self._last_seen[r]
                if step > seen_step:
                    self._last_seen[r] = (step, now)
                elif step < self._my_step and now - since > self.timeout_s:
                    # the peer is behind this rank and has not moved for longer than the limit
                    self._failure = PeerFailure("HANG", r, f"no progress past step {step // 2} for {now - since:.1f} s "
                                                           f"(this rank is in step {(self._my_step + 1) // 2})")
                    return
            self._stop.wait(self.poll_s)
