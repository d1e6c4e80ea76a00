"""Tracing helpers: NVTX ranges around every collective and an optional host-side phase profiler.

Environment:
    DEEPEP_PROFILE=1            enable :class:`PhaseProfiler` printing (averaged per-phase milliseconds on stderr)
    DEEPEP_PROFILE_INTERVAL=N   print every N iterations (default 50)
    DEEPEP_PROFILE_WARMUP=N     ignore the first N iterations (default 10)

Reference counterpart: ``_LLProfiler`` (deep_ep/buffer.py:16-77), which synchronises the device at every
mark. This one records CUDA events instead and resolves them when an iteration is finished, so enabling
it does not serialise the pipeline.
"""
from __future__ import annotations

import contextlib
import os
import sys
from collections import defaultdict
from typing import Dict, List, Tuple

import torch

PROFILE_ENABLED = os.environ.get("DEEPEP_PROFILE", "0") == "1"
PROFILE_INTERVAL = int(os.environ.get("DEEPEP_PROFILE_INTERVAL", "50"))
PROFILE_WARMUP = int(os.environ.get("DEEPEP_PROFILE_WARMUP", "10"))

_NVTX = os.environ.get("DEEPEP_NVTX", "0") == "1"


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range when ``DEEPEP_NVTX=1`` and CUDA is present; otherwise free."""
    if _NVTX and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class PhaseProfiler:
    """Per-phase device timing: ``mark(name)`` records an event; ``finish_iter()`` closes an iteration."""

    def __init__(self, title: str, rank: int, interval: int = PROFILE_INTERVAL, warmup: int = PROFILE_WARMUP,
                 stream=sys.stderr) -> None:
        self.title, self.rank, self.interval, self.warmup, self.stream = title, rank, interval, warmup, stream
        self.marks: List[Tuple[str, "torch.cuda.Event"]] = []
        self.pending: List[List[Tuple[str, "torch.cuda.Event"]]] = []
        self.totals: Dict[str, float] = defaultdict(float)
        self.iters = 0
        self.counted = 0

    def mark(self, name: str) -> None:
        if not torch.cuda.is_available():
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.marks.append((name, ev))

    def finish_iter(self) -> None:
        self.iters += 1
        if self.iters > self.warmup and self.marks:
            self.pending.append(self.marks)
        self.marks = []
        if self.pending and len(self.pending) >= self.interval:
            self.flush()

    def flush(self) -> Dict[str, float]:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        for marks in self.pending:
            for (_, a), (name, b) in zip(marks[:-1], marks[1:]):
                self.totals[name] += a.elapsed_time(b)
            self.counted += 1
        self.pending = []
        avg = {k: v / max(self.counted, 1) for k, v in self.totals.items()}
        if avg:
            line = " ".join(f"{k}={v * 1e3:.1f}us" for k, v in avg.items())
            print(f"[{self.title} r{self.rank}] n={self.counted} {line}", file=self.stream, flush=True)
        return avg
