"""Opt-in tracing: NVTX ranges around layers / phases, host-side phase timers for `/metrics`, and a
`torch.profiler` context for one-off traces.  Everything is off unless `SLOPLLM_B200_NVTX=1` (ranges)
or the caller asks (timers, profiler), so the hot path pays one attribute test.

Reference: `recordPhase` (`src/generation-scheduler.ts:438-447`), `profilerStart/Stop`
(`csrc/glm_ops.cpp`); the reference has no NVTX ranges.
"""
from __future__ import annotations

import functools
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


def traced(label):
    """Method decorator: an NVTX range around every call while `SLOPLLM_B200_NVTX=1` (otherwise one module attribute
    test per call).  `label` is the range name, or a function of the call's arguments that returns it."""
    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*a, **k):
            if not NVTX:
                return fn(*a, **k)
            with nvtx_range(label(*a, **k) if callable(label) else label):
                return fn(*a, **k)
        return wrapper
    return deco


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


class OpTimers:
    """Device time per backend op: wraps the public methods of an ops object with CUDA event pairs.

    Eager mode only (events cannot be recorded inside a graph capture).  Each rank of a multi-GPU job
    can carry its own instance, which is how a per-op breakdown of a multi-rank step is taken without
    a profiler.  `summary()` synchronises once and returns rows sorted by total time."""

    def __init__(self, ops, names=None):
        self.ops = ops
        self.events = defaultdict(list)
        self._orig = {}
        self._depth = 0
        self._others = []
        self.attach(ops, names)

    def attach(self, obj, names=None, prefix: str = "") -> None:
        """Time another object's public methods under the same nesting rule (e.g. the communicator next to the ops:
        a collective that calls a backend op inside counts once, as the collective)."""
        names = names or [n for n in dir(obj) if not n.startswith("_") and callable(getattr(obj, n, None))
                          and n not in ("name",)]
        for n in names:
            fn = getattr(obj, n)
            if isinstance(fn, type) or not hasattr(fn, "__call__"):
                continue
            if obj is self.ops:
                self._orig[n] = fn
            else:
                self._others.append((obj, n, fn))
            setattr(obj, n, self._wrap(prefix + n, fn))

    def _wrap(self, name, fn):
        def timed(*a, **k):
            if self._depth > 0 or not torch.cuda.is_available():      # nested backend calls count towards the outer op
                return fn(*a, **k)
            self._depth += 1
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            try:
                return fn(*a, **k)
            finally:
                e1.record()
                self.events[name].append((e0, e1))
                self._depth -= 1
        return timed

    def reset(self) -> None:
        self.events.clear()

    def restore(self) -> None:
        for n, fn in self._orig.items():
            setattr(self.ops, n, fn)
        self._orig.clear()
        for obj, n, fn in self._others:
            setattr(obj, n, fn)
        self._others.clear()

    def summary(self):
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        rows = []
        for n, evs in self.events.items():
            ms = sum(a.elapsed_time(b) for a, b in evs)
            rows.append({"op": n, "calls": len(evs), "total_ms": round(ms, 4), "us_per_call": round(1e3 * ms / max(1, len(evs)), 2)})
        rows.sort(key=lambda r: -r["total_ms"])
        tot = sum(r["total_ms"] for r in rows) or 1.0
        for r in rows:
            r["share"] = round(r["total_ms"] / tot, 4)
        return rows
