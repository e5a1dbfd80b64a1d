"""Rank-failure detection on the host, and host-side fault injection for its tests.

Every rank runs a `HealthMonitor`: a daemon thread that writes a heartbeat into a shared key-value
store (`torch.distributed.TCPStore`, hosted by rank 0) and reads the peers' heartbeats.  A peer whose
heartbeat is older than `timeout_s` marks this rank unhealthy: `/health` answers 503, the scheduler
fails in-flight requests fast instead of launching a collective that could never complete, and the
`on_failure` callback lets the process re-initialise its communicators (the weights stay with the
loader process).  Device-side waits are bounded separately (`CollectiveTimeout`, parallel/nvlink.py);
this module never touches a GPU.

The reference has no counterpart (single process; its P2P barrier spins without bound,
`csrc/glm_p2p.cu:180`); its only failure handling is the scheduler's per-batch rollback and
`isFatalCudaError` (`src/generation-scheduler.ts:63-66, 669-689`).
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional


@dataclass
class HealthState:
    healthy: bool = True
    failed_ranks: List[int] = field(default_factory=list)
    reason: str = ""
    since: float = 0.0


class HealthMonitor:
    def __init__(self, store, rank: int, world: int, interval_s: float = 0.2, timeout_s: float = 2.0,
                 on_failure: Optional[Callable[[HealthState], None]] = None, clock: Callable[[], float] = time.time):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s = interval_s, timeout_s
        self.on_failure = on_failure
        self.clock = clock
        self.state = HealthState()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._paused = False                      # fault injection: stop beating without stopping the thread
        self._last_seen: Dict[int, float] = {}
        self.beats = 0

    # -- lifecycle ---------------------------------------------------------------------------------------
    def start(self) -> "HealthMonitor":
        self.beat()
        self._thread = threading.Thread(target=self._run, name=f"health-{self.rank}", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)

    # -- heartbeat -----------------------------------------------------------------------------------------
    def beat(self) -> None:
        if not self._paused:
            self.beats += 1
            self.store.set(f"hb/{self.rank}", repr(self.clock()))

    def pause(self) -> None:
        """Host-side fault injection: this rank keeps running but stops sending heartbeats."""
        self._paused = True

    def check_peers(self) -> HealthState:
        now = self.clock()
        failed = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                ts = float(self.store.get(f"hb/{r}").decode())
                self._last_seen[r] = ts
            except Exception:  # noqa: BLE001  (key missing yet, or the store host is gone)
                ts = self._last_seen.get(r)
                if ts is None:
                    self._last_seen[r] = ts = now       # grace period from the first look
            if now - ts > self.timeout_s:
                failed.append(r)
        if failed and self.state.healthy:
            self.state = HealthState(False, failed, f"no heartbeat from rank(s) {failed} for more than {self.timeout_s} s", now)
            if self.on_failure is not None:
                self.on_failure(self.state)
        return self.state

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            try:
                self.beat()
            except Exception:  # noqa: BLE001  (store host died: peers will notice, and so will check_peers)
                pass
            self.check_peers()

    def is_healthy(self) -> bool:
        return self.state.healthy

    def raise_if_unhealthy(self) -> None:
        """Call before launching a step: a dead peer would leave the step's collectives waiting."""
        if not self.state.healthy:
            raise RankFailure(self.state.reason)

    def reset(self) -> None:
        """After the communicators were rebuilt without the failed ranks (or with replacements)."""
        self.state = HealthState()
        self._last_seen.clear()


class RankFailure(RuntimeError):
    pass


class FaultInjector:
    """Deterministic host-side faults for tests: named sites count down and then raise / drop."""

    def __init__(self):
        self._arm: Dict[str, int] = {}
        self.fired: List[str] = []

    def arm(self, site: str, after: int = 0) -> None:
        self._arm[site] = after

    def hit(self, site: str) -> bool:
        """True when the fault at `site` fires now."""
        if site not in self._arm:
            return False
        if self._arm[site] > 0:
            self._arm[site] -= 1
            return False
        del self._arm[site]
        self.fired.append(site)
        return True

    def maybe_raise(self, site: str, exc: Exception) -> None:
        if self.hit(site):
            raise exc


def make_store(rank: int, world: int, host: str = "127.0.0.1", port: int = 29600, timeout_s: float = 30.0):
    """TCPStore hosted by rank 0 (127.0.0.1 by default: container hostnames may not resolve)."""
    from datetime import timedelta

    import torch.distributed as dist
    return dist.TCPStore(host, port, world, is_master=(rank == 0), timeout=timedelta(seconds=timeout_s), wait_for_workers=False)
