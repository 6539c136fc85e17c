"""torch.profiler capture of a window of training steps, one Kineto trace per profiled rank.

Knobs mirror the reference's profiler enablement (``.cursor/skills/gpu-trace-analysis/SKILL.md:141-168``):
``profile``, ``profile_step_start/end``, ``profile_ranks``, stacks and shapes off by default (shapes at
8 ranks ran the reference out of memory).  Each step is wrapped in a ``ProfilerStep#N`` annotation so
the analyzer can pick a window.
"""
from __future__ import annotations

from pathlib import Path

import torch


class StepProfiler:
    def __init__(self, pcfg, rank: int):
        self.cfg, self.rank = pcfg, rank
        self.prof = None
        self.range = None
        self.path = None

    def step_begin(self, step: int) -> None:
        c = self.cfg
        if step == c.profile_step_start and self.prof is None:
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self.prof = torch.profiler.profile(activities=acts, with_stack=c.torch_profiler_with_stack,
                                               record_shapes=c.torch_profiler_record_shapes)
            self.prof.__enter__()
        if self.prof is not None:
            self.range = torch.profiler.record_function(f"ProfilerStep#{step}")
            self.range.__enter__()

    def step_end(self, step: int) -> None:
        if self.prof is None:
            return
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        if self.range is not None:
            self.range.__exit__(None, None, None)
            self.range = None
        if step >= self.cfg.profile_step_end:
            self.prof.__exit__(None, None, None)
            out = Path(self.cfg.trace_dir)
            out.mkdir(parents=True, exist_ok=True)
            self.path = str(out / f"rank{self.rank}_steps{self.cfg.profile_step_start}-{step}.pt.trace.json")
            self.prof.export_chrome_trace(self.path)
            self.prof = None
