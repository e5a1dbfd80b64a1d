"""CUDA-graph cache for fixed-shape steps.

Parity: `src/capture-manager.ts:29-301` keys graphs by caller parameters + batch size +
token count + KV-length bucket, runs the first calls of a key eagerly as warm-up, then
captures and replays.  Here a key maps to a `torch.cuda.CUDAGraph` whose inputs and outputs
are static tensors owned by the entry; `SLOPLLM_B200_CAPTURE_DEBUG=1` prints key activity.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Hashable, Optional

import torch

from ..config import env_flag, env_int


@dataclass
class GraphEntry:
    calls: int = 0
    graph: Optional[Any] = None
    outputs: Any = None
    launches: int = 0                 # native library calls recorded while capturing
    kernels: int = 0                  # CUDA kernels of the library recorded while capturing (a call may launch several)
    extra: dict = field(default_factory=dict)


class CaptureManager:
    def __init__(self, enabled: bool = True, warmups: Optional[int] = None):
        self.enabled = enabled and torch.cuda.is_available()
        self.warmups = env_int("CAPTURE_WARMUPS", 1) if warmups is None else warmups
        self.debug = env_flag("CAPTURE_DEBUG")
        self.entries: Dict[Hashable, GraphEntry] = {}
        self.pool = None

    def execute(self, key: Hashable, fn: Callable[[], Any]) -> Any:
        """Run `fn` (which reads only static input tensors and returns static outputs):
        eagerly for the first `warmups` calls of `key`, captured on the next, replayed after."""
        if not self.enabled:
            return fn()
        e = self.entries.setdefault(key, GraphEntry())
        e.calls += 1
        if e.graph is not None:
            e.graph.replay()
            return e.outputs
        if e.calls <= self.warmups:
            if self.debug:
                print(f"[capture] warm-up {e.calls}/{self.warmups} key={key}")
            return fn()
        from ..ops import native as N
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        if self.pool is None:
            self.pool = torch.cuda.graph_pool_handle()
        before, kbefore = N.launch_count(), N.kernel_count()
        # Collected garbage may own CUDA graphs or memory pools of engines that are gone; destroying those while a
        # capture is open invalidates it.  Collect now, and keep the collector off until the capture has ended.
        import gc
        gc.collect()
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(g, pool=self.pool):
                e.outputs = fn()
        finally:
            if gc_was_on:
                gc.enable()
        e.launches = N.launch_count() - before
        e.kernels = N.kernel_count() - kbefore
        e.graph = g
        if self.debug:
            print(f"[capture] captured key={key} library calls={e.launches} kernels={e.kernels}")
        g.replay()
        return e.outputs

    def launches_for(self, key: Hashable) -> int:
        e = self.entries.get(key)
        return e.launches if e else 0

    def uncapture(self, key: Optional[Hashable] = None) -> None:
        if key is None:
            self.entries.clear()
        else:
            self.entries.pop(key, None)
