"""Lock-step scheduling across the ranks of one model replica.

Every rank runs the same `GenerationScheduler` over its shard of the model.  Rank 0 owns the
HTTP front end; before each step it broadcasts what arrived since the last one (new requests,
cancellations, cache flushes, stop) and every rank applies exactly that, so admission, batching
and retirement are identical everywhere and the collectives inside the model line up.  Sampling
is deterministic per (seed, row, step), so the ranks also agree on every token.

The reference runs all GPUs from one process and has no counterpart; the broadcast replaces its
single `GenerationScheduler` event queue (`src/generation-scheduler.ts:357-420`).
"""
from __future__ import annotations

import queue
from dataclasses import asdict
from typing import Dict, List, Optional

import torch.distributed as dist

from ..config import SamplingParams
from .scheduler import CacheFlushEvent, GenerationRequest


class ReplicaChannel:
    def __init__(self, rank: int, world: int, group=None, idle_wait_s: float = 0.02, src: int = 0):
        self.rank, self.world, self.group = rank, world, group
        self.src = src                                          # job-wide rank of this replica's rank 0
        self.idle_wait_s = idle_wait_s
        self.live: Dict[str, GenerationRequest] = {}          # requests known to this rank, by id
        self.inbox: "queue.Queue" = queue.Queue()             # rank 0: what the front end submitted since the last step
        self._local_objects = {"requests": [], "flush": []}

    # ---- rank 0: collect, everyone: apply -------------------------------------------------------------
    def _collect(self, sched) -> dict:
        items: List[object] = []
        try:
            if not sched.rows and sched.events.empty():
                items.append(self.inbox.get(timeout=self.idle_wait_s))
            while True:
                items.append(self.inbox.get_nowait())
        except queue.Empty:
            pass
        wire = {"requests": [], "flush": [], "stop": False, "cancel": []}
        self._local_objects = {"requests": [], "flush": []}
        for ev in items:
            if ev is None:
                wire["stop"] = True
            elif isinstance(ev, CacheFlushEvent):
                wire["flush"].append(ev.kind)
                self._local_objects["flush"].append(ev)
            else:
                wire["requests"].append({"id": ev.id, "input_ids": list(ev.input_ids), "max_tokens": ev.max_tokens,
                                         "sampling": asdict(ev.sampling), "stop_token_ids": list(ev.stop_token_ids)})
                self._local_objects["requests"].append(ev)
        wire["cancel"] = [rid for rid, r in self.live.items() if r.cancelled and not r.cancel_seen]
        wire["cancel"] += [r.id for r in self._local_objects["requests"] if r.cancelled]
        return wire

    def exchange(self, sched) -> None:
        payload = [self._collect(sched) if self.rank == 0 else None]
        if self.world > 1:
            dist.broadcast_object_list(payload, src=self.src, group=self.group)
        wire = payload[0]
        if wire["stop"]:
            self._drop_retired()
            sched._stop.set()
            return
        for i, kind in enumerate(wire["flush"]):
            sched.events.put(self._local_objects["flush"][i] if self.rank == 0 else CacheFlushEvent(kind))
        for i, d in enumerate(wire["requests"]):
            if self.rank == 0:
                req = self._local_objects["requests"][i]
            else:
                req = GenerationRequest(id=d["id"], input_ids=d["input_ids"], max_tokens=d["max_tokens"],
                                        sampling=SamplingParams(**d["sampling"]), stop_token_ids=d["stop_token_ids"])
            self.live[req.id] = req
            sched.events.put(req)
        for rid in wire["cancel"]:
            r = self.live.get(rid)
            if r is not None:
                r.cancelled = r.cancel_seen = True
        self._drop_retired()

    def _drop_retired(self) -> None:
        """A request leaves the table when the scheduler has retired it, not when a finish reason appears: until then a
        cancellation of it may still have to travel to the other ranks."""
        for rid in [rid for rid, r in self.live.items() if r.retired]:
            del self.live[rid]


def make_channel(ctx, idle_wait_s: float = 0.02) -> Optional[ReplicaChannel]:
    """A channel over a dedicated gloo group of this replica's ranks when the replica has more than one rank.  Under data
    parallelism every rank of the job creates every replica's group (group creation is collective over the job)."""
    if not dist.is_initialized() or (ctx.world <= 1 and ctx.dp_world <= 1):
        return None
    if ctx.dp_world <= 1:
        return ReplicaChannel(ctx.rank, ctx.world, dist.new_group(backend="gloo"), idle_wait_s)
    mine = None
    for d in range(ctx.dp_world):
        g = dist.new_group(ranks=list(range(d * ctx.world, (d + 1) * ctx.world)), backend="gloo")
        if d == ctx.dp_rank:
            mine = g
    if ctx.world <= 1:
        return None
    return ReplicaChannel(ctx.rank, ctx.world, mine, idle_wait_s, src=ctx.dp_rank * ctx.world)
