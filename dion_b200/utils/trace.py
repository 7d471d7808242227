"""Named ranges for profilers.

``with trace.span("name"):`` pushes an NVTX range (visible in Nsight Systems / Nsight Compute
and in ``torch.profiler`` traces) around a phase of the optimizer or training step.  Ranges cost
nothing unless tracing is on: set ``DION_B200_NVTX=1`` or call ``trace.enable()``.  The reference
has no tracing hooks; its only instrumentation is wall-clock timing in train.py:1013-1059.

``trace.profile_steps(step_fn, n, path)`` runs ``n`` calls of ``step_fn`` under ``torch.profiler``
(CPU + CUDA activities), writes a Chrome trace to ``path`` and returns the per-kernel table as a
string.
"""
from __future__ import annotations

import os
from typing import Callable, Optional

import torch

_enabled = os.environ.get("DION_B200_NVTX", "0") == "1"


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled


class _Range:
    __slots__ = ("name", "active")

    def __init__(self, name: str):
        self.name = name
        self.active = False

    def __enter__(self):
        if _enabled and torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.name)
            self.active = True
        return self

    def __exit__(self, *exc):
        if self.active:
            torch.cuda.nvtx.range_pop()
            self.active = False
        return False


def span(name: str) -> _Range:
    return _Range(name)


def mark(name: str) -> None:
    if _enabled and torch.cuda.is_available():
        torch.cuda.nvtx.mark(name)


def profile_steps(step_fn: Callable[[], object], steps: int, trace_path: Optional[str] = None,
                  row_limit: int = 40) -> str:
    """Profile ``steps`` calls of ``step_fn``; returns the kernel table sorted by device time."""
    from torch.profiler import ProfilerActivity, profile

    acts = [ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(ProfilerActivity.CUDA)
    was = _enabled
    enable(True)
    try:
        with profile(activities=acts) as prof:
            for _ in range(steps):
                step_fn()
            if torch.cuda.is_available():
                torch.cuda.synchronize()
    finally:
        enable(was)
    if trace_path:
        prof.export_chrome_trace(trace_path)
    key = "cuda_time_total" if torch.cuda.is_available() else "cpu_time_total"
    return prof.key_averages().table(sort_by=key, row_limit=row_limit)

