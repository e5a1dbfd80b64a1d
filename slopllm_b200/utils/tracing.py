"""Opt-in tracing: NVTX ranges around layers / phases, host-side phase timers for `/metrics`, and a
`torch.profiler` context for one-off traces.  Everything is off unless `SLOPLLM_B200_NVTX=1` (ranges)
or the caller asks (timers, profiler), so the hot path pays one attribute test.

Reference: `recordPhase` (`src/generation-scheduler.ts:438-447`), `profilerStart/Stop`
(`csrc/glm_ops.cpp`); the reference has no NVTX ranges.
"""
from __future__ import annotations

import os
import time
from collections import defaultdict
from contextlib import contextmanager
from typing import Dict, Iterator, Tuple

import torch

NVTX = os.environ.get("SLOPLLM_B200_NVTX", "0") == "1"


@contextmanager
def nvtx_range(name: str) -> Iterator[None]:
    if NVTX and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class PhaseTimers:
    """seconds / count per (phase, batch size), exported by the server as `slopllm:phase_seconds_*`."""

    def __init__(self):
        self.seconds: Dict[Tuple[str, int], float] = defaultdict(float)
        self.count: Dict[Tuple[str, int], int] = defaultdict(int)

    def record(self, phase: str, batch_size: int, seconds: float) -> None:
        self.seconds[(phase, batch_size)] += seconds
        self.count[(phase, batch_size)] += 1

    @contextmanager
    def phase(self, name: str, batch_size: int = 0) -> Iterator[None]:
        t0 = time.perf_counter()
        with nvtx_range(name):
            yield
        self.record(name, batch_size, time.perf_counter() - t0)

    def prometheus(self, prefix: str = "slopllm") -> str:
        lines = []
        for (phase, b), s in sorted(self.seconds.items()):
            lines.append(f'{prefix}:phase_seconds_sum{{phase="{phase}",batch_size="{b}"}} {s:.6f}')
            lines.append(f'{prefix}:phase_seconds_count{{phase="{phase}",batch_size="{b}"}} {self.count[(phase, b)]}')
        return "\n".join(lines) + ("\n" if lines else "")


@contextmanager
def torch_profile(path: str, cuda: bool = True) -> Iterator[None]:
    """Chrome trace of the enclosed region (`chrome://tracing`, Perfetto)."""
    acts = [torch.profiler.ProfilerActivity.CPU]
    if cuda and torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    with torch.profiler.profile(activities=acts) as prof:
        yield
    prof.export_chrome_trace(path)
