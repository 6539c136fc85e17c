"""MLPerf-style event lines (``:::MLLOG {json}``) and the final ``RESULT`` line.

Event keys follow what the reference's runs emitted
(``notes/2026-04/2026-04-19_gptoss_01_mlperf_best_e2e_run.md:33-54``,
``notes/2026-04/2026-04-28_gptoss_27_mlperf_legal_baseline.md:62-67,179-189``):
``run_start``, ``run_stop``, ``run_duration``, ``eval_accuracy``, ``samples_count``.
"""
from __future__ import annotations

import json
import sys
import time


class MLLogger:
    def __init__(self, enabled: bool = True, benchmark: str = "moe_pretraining", org: str = "system_lab_b200",
                 stream=None):
        self.enabled, self.benchmark, self.org = enabled, benchmark, org
        self.stream = stream or sys.stdout
        self.t0 = None

    def event(self, key: str, value=None, **meta) -> None:
        if not self.enabled:
            return
        rec = {"namespace": "", "time_ms": int(time.time() * 1e3), "event_type": "POINT_IN_TIME",
               "key": key, "value": value, "metadata": meta}
        print(":::MLLOG " + json.dumps(rec), file=self.stream, flush=True)

    def start(self, cfg) -> None:
        self.t0 = time.time()
        self.event("global_batch_size", cfg.train.global_batch_size)
        self.event("seed", cfg.train.seed)
        self.event("run_start", None, status="running")

    def eval(self, value: float, samples: int) -> None:
        self.event("eval_accuracy", value, samples_count=samples)

    def stop(self, samples: int, status: str = "success") -> None:
        dur = time.time() - (self.t0 or time.time())
        self.event("samples_count", samples)
        self.event("run_stop", None, status=status)
        self.event("run_duration", dur)
        if self.enabled:
            print(f"RESULT,{self.benchmark},,{int(dur)},{self.org},{time.strftime('%Y-%m-%d %I:%M:%S %p')}",
                  file=self.stream, flush=True)
