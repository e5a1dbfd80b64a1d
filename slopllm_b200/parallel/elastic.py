"""Rebuilding the process group after a rank has been lost, without restarting the survivors.

A `torch.distributed` process group cannot shrink or take a replacement member, so recovery means a new group.
Every incarnation of the group is a *generation*: all members rendezvous through one long-lived key-value store
(`TCPStore`; hosted by rank 0, or by the persistent loader process, which outlives executors) under the prefix
`gen<N>/`, so keys of a dead generation can never satisfy a later rendezvous.

    survivors   notice the failure on the host (`utils/health.py`: a stale heartbeat, or a collective that raised
                after its process-group timeout), stop launching work, and call `ElasticGroup.recover()`;
                the first of them advances the store's `elastic/generation` counter
    replacement a fresh process for the lost rank calls `ElasticGroup.join()`: it looks up the newest generation its
                rank number was a member of (every member records itself in the store), waits for a newer one and
                enters it
    everyone    tears down its old group locally and runs `init_process_group` on the generation's prefix; the
                call returns once all `world` members of that generation have arrived

What lives on top of the group is rebuilt by the caller from the returned `ParallelContext`: `make_comm` allocates and
maps a fresh symmetric region (the old peer mappings point into a dead process), the engine drops its CUDA graphs (they
captured collectives of the old communicator) and the scheduler re-queues or fails the requests that were in flight.
The weights are untouched: sharded weights stay on the survivors' GPUs, and a replacement maps the loader's copy.

A rank leaves only between steps in the tests of this module (no kernel or collective in flight), and they run on gloo
CPU ranks.  The reference has no counterpart (one process drives all GPUs; a lost GPU ends the server, which Docker
restarts: `docker-compose.yml`, `src/generation-scheduler.ts:63-66`).
"""
from __future__ import annotations

import time
from datetime import timedelta
from typing import Callable, Optional

import torch
import torch.distributed as dist

from .dist import ParallelContext

GENERATION_KEY = "elastic/generation"


class RecoveryTimeout(RuntimeError):
    """The members of the new generation did not all arrive in time."""


class ElasticGroup:
    """One rank's handle on the generations of its process group."""

    def __init__(self, store, rank: int, world: int, device: Optional[torch.device] = None, backend: Optional[str] = None,
                 cp: bool = False, ep: bool = False, timeout_s: float = 60.0):
        self.store, self.rank, self.world = store, rank, world
        self.device = device or torch.device("cpu")
        self.backend = backend or ("nccl" if self.device.type == "cuda" else "gloo")
        self.cp, self.ep, self.timeout_s = cp, ep, timeout_s
        self.generation = -1
        self._tried = -1              # newest generation this rank entered or tried to enter
        self.ctx: Optional[ParallelContext] = None

    # -- generation counter ------------------------------------------------------------------------------------
    def current_generation(self) -> int:
        """The store's counter (0 before any recovery); `add(key, 0)` reads it without a separate existence check."""
        return int(self.store.add(GENERATION_KEY, 0))

    def _enter(self, generation: int) -> ParallelContext:
        self._leave()
        self._tried = max(self._tried, generation)
        # c10d names the default group's rendezvous keys after a per-process group counter that a *failed*
        # init_process_group leaves advanced; a process that has tried before must count like one that has not
        world_state = getattr(dist.distributed_c10d, "_world", None)
        if world_state is not None and not dist.is_initialized():
            world_state.group_count = 0
        prefix = dist.PrefixStore(f"gen{generation}/", self.store)
        kw = {"device_id": self.device} if self.device.type == "cuda" else {}
        try:
            dist.init_process_group(self.backend, store=prefix, rank=self.rank, world_size=self.world,
                                    timeout=timedelta(seconds=self.timeout_s), **kw)
        except Exception as e:  # noqa: BLE001  (c10d raises DistStoreError / RuntimeError on a rendezvous that timed out)
            # the attempt's rendezvous keys stay under this prefix: nobody may try to assemble this generation again
            self.store.set(f"elastic/spent/{generation}", "1")
            raise RecoveryTimeout(f"rank {self.rank}: generation {generation} did not assemble within {self.timeout_s} s: {e}") from e
        self.generation = generation
        self.store.set(f"elastic/member/{generation}/{self.rank}", "1")
        self.ctx = ParallelContext(self.rank, self.world, self.device, self.cp, self.ep, dist.group.WORLD if self.world > 1 else None)
        return self.ctx

    def _leave(self) -> None:
        """Drop the current group locally.  Peers may be gone, so nothing here may wait for them: NCCL communicators
        are aborted where torch offers it, otherwise destroyed."""
        if not dist.is_initialized():
            return
        abort = getattr(dist.distributed_c10d, "_abort_process_group", None)
        try:
            if self.backend == "nccl" and abort is not None:
                abort()
            else:
                dist.destroy_process_group()
        except Exception:  # noqa: BLE001  (a half-dead group may refuse a clean shutdown; the new generation does not need it)
            pass

    # -- entry points --------------------------------------------------------------------------------------------
    def start(self) -> ParallelContext:
        """First start of the job: every rank enters the store's current generation (0 on a fresh store)."""
        return self._enter(self.current_generation())

    def join(self) -> ParallelContext:
        """A replacement process for a lost rank: find the newest generation that this rank number was a member of
        (its predecessor's, which is dead), wait until the survivors have opened a newer one, and enter it."""
        dead = -1
        for g in range(self.current_generation(), -1, -1):
            if self.store.check([f"elastic/member/{g}/{self.rank}"]):
                dead = g
                break
        # a generation whose assembly already failed for somebody is skipped: the survivors will open another one
        while True:
            g = self._wait_for_generation_above(dead)
            if self.store.check([f"elastic/spent/{g}"]):
                dead = g
                continue
            return self._enter(g)

    def recover(self, on_new_context: Optional[Callable[[ParallelContext], None]] = None) -> ParallelContext:
        """A survivor: open a generation that nobody has tried yet and enter it.  Every entrant (survivors here, a
        replacement in `join`) enters the value of the store's counter, so they cannot end up in different generations.
        The counter is moved by one rank only: the first to claim the next number (an `add` on a per-number claim key).
        After a `RecoveryTimeout` the generation that failed to assemble is spent (its prefix still holds the rendezvous
        keys of the attempt): the next call opens a fresh one.  `on_new_context` rebuilds what was attached to the old
        group (communicator, graphs)."""
        tried = max(self._tried, self.generation)
        cur = self.current_generation()
        if cur <= tried:
            nxt = tried + 1
            # one claim key per generation: the first `add` returns 1 and that rank advances the counter to it
            if int(self.store.add(f"elastic/claim/{nxt}", 1)) == 1:
                cur = self.current_generation()
                if cur < nxt:
                    self.store.add(GENERATION_KEY, nxt - cur)
        gen = self._wait_for_generation_above(tried)
        ctx = self._enter(gen)
        if on_new_context is not None:
            on_new_context(ctx)
        return ctx

    def _wait_for_generation_above(self, g: int) -> int:
        deadline = time.time() + self.timeout_s
        while True:
            cur = self.current_generation()
            if cur > g:
                return cur
            if time.time() > deadline:
                raise RecoveryTimeout(f"rank {self.rank}: no generation above {g} was opened within {self.timeout_s} s")
            time.sleep(0.05)

    def shutdown(self) -> None:
        self._leave()
        self.ctx = None


def reattach(engine, ctx: ParallelContext, cfg=None, fused: bool = True) -> None:
    """Point a running engine at a new generation's context: a fresh communicator for the model (on CUDA this allocates
    and maps a new symmetric region; the old mappings pointed into the lost process), and no CUDA graph of the old
    generation survives, because graphs captured that generation's collectives.  Weights, KV cache and scheduler state
    stay as they are; the caller decides what happens to the requests that were in flight."""
    from .fused import make_comm
    model = engine.model
    old = getattr(model, "comm", None)
    if old is not None and hasattr(old, "close"):
        old.close()                       # peer mappings of the previous generation
    model.ctx = ctx
    model.comm = make_comm(ctx, cfg if cfg is not None else getattr(model, "cfg", None), fused=fused)
    if getattr(model, "ops", None) is not None and hasattr(model.ops, "ctx"):
        model.ops.ctx = ctx
    graphs = getattr(engine, "graphs", None)
    if graphs is not None:
        graphs.uncapture()
