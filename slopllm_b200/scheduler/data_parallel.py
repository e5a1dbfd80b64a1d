"""Data parallelism for serving: several model replicas behind one front end.

A job of W ranks started with `--dp D` forms D replicas of W / D ranks (tensor / context / expert parallel inside a
replica, as without `--dp`).  Every replica runs its own `GenerationScheduler` with its own KV cache and prefix cache;
replicas never exchange activations, so they run at their own pace.  The HTTP front end lives on job rank 0 and talks to

* its own replica's scheduler directly, and
* every other replica through a pair of ordered mailboxes on the job's key-value store (`TCPStore`): requests,
  cancellations and cache flushes go to the replica's first rank (`ReplicaAgent`), token batches, completions and metric
  snapshots come back (`ReplicaProxy`).  The traffic is a few dozen bytes per generated token, far below what the store
  handles; the model's collectives never touch it.

`DataParallelRouter` offers the front end the scheduler's interface (`submit`, `flush_*_cache`, `metrics`, `engine.kv`)
and places each request on the replica with the fewest live requests, except that a prompt whose first KV page was seen
before goes back to the replica that served it (its prefix cache holds those pages) unless that replica is clearly busier.

The reference has one model replica per server (`src/generation-scheduler.ts`); this module has no counterpart there.
"""
from __future__ import annotations

import pickle
import threading
import time
from dataclasses import asdict, fields
from types import SimpleNamespace
from typing import Dict, List, Optional

from ..config import SamplingParams
from .scheduler import CacheFlushEvent, GenerationRequest, ServerMetrics


class Mailbox:
    """Ordered multi-producer / single-consumer queue on a key-value store: `put` takes the next sequence number and
    stores the message under it; `drain` returns the messages that have been numbered since the last call, in order."""

    def __init__(self, store, name: str):
        self.store, self.name = store, name
        self._read = 0

    def put(self, obj) -> None:
        seq = int(self.store.add(f"{self.name}/n", 1))
        self.store.set(f"{self.name}/{seq}", pickle.dumps(obj))

    def wait_next(self, timeout_s: float) -> bool:
        """Block until the next message has been stored, or `timeout_s` has passed (False)."""
        from datetime import timedelta
        try:
            self.store.wait([f"{self.name}/{self._read + 1}"], timedelta(seconds=timeout_s))
            return True
        except Exception:  # noqa: BLE001  (the store raises on a wait that ran out)
            return False

    def drain(self) -> List[object]:
        n = int(self.store.add(f"{self.name}/n", 0))
        out = []
        while self._read < n:
            key = f"{self.name}/{self._read + 1}"
            out.append(pickle.loads(self.store.get(key)))       # blocks (store timeout) until the producer's `set` lands
            self.store.delete_key(key)
            self._read += 1
        return out


def _wire_request(req: GenerationRequest) -> dict:
    return {"op": "submit", "id": req.id, "input_ids": list(req.input_ids), "max_tokens": req.max_tokens,
            "sampling": asdict(req.sampling), "stop_token_ids": list(req.stop_token_ids)}


_RESULT_FIELDS = ("finish_reason", "error", "prompt_tokens", "cached_tokens", "prefill_tokens", "prefill_seconds")


class ReplicaAgent:
    """Runs on the first rank of a replica other than the front end's: feeds the local scheduler from the replica's
    inbox and reports tokens, completions and metrics to its outbox."""

    def __init__(self, store, replica: int, scheduler, poll_s: float = 0.005, metrics_every_s: float = 0.5):
        self.inbox, self.outbox = Mailbox(store, f"dp/{replica}/in"), Mailbox(store, f"dp/{replica}/out")
        self.sched, self.poll_s, self.metrics_every_s = scheduler, poll_s, metrics_every_s
        self.live: Dict[str, GenerationRequest] = {}
        self._pending: Dict[str, List[int]] = {}                 # tokens produced since the last report, by request
        self._done: List[GenerationRequest] = []
        self._flushes: List[tuple] = []
        self._lock = threading.Lock()
        self._wake = threading.Event()                           # set by the scheduler thread when there is something to report
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def start(self) -> "ReplicaAgent":
        self._thread = threading.Thread(target=self._run, name="dp-agent", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)

    # scheduler-thread callbacks: only touch the buffers
    def _on_token(self, rid: str, tok: int) -> None:
        with self._lock:
            self._pending.setdefault(rid, []).append(int(tok))
        self._wake.set()

    def _on_finish(self, req: GenerationRequest) -> None:
        with self._lock:
            self._done.append(req)
        self._wake.set()

    def _handle(self, msg: dict) -> bool:
        op = msg["op"]
        if op == "submit":
            rid = msg["id"]
            req = GenerationRequest(id=rid, input_ids=msg["input_ids"], max_tokens=msg["max_tokens"],
                                    sampling=SamplingParams(**msg["sampling"]), stop_token_ids=msg["stop_token_ids"],
                                    on_token=lambda t, rid=rid: self._on_token(rid, t), on_finish=self._on_finish)
            self.live[rid] = req
            self.sched.submit(req)
        elif op == "cancel":
            req = self.live.get(msg["id"])
            if req is not None:
                req.cancel()
        elif op == "flush":
            ev = self.sched.flush_gpu_cache() if msg["kind"] == "flush_gpu_cache" else self.sched.flush_host_cache()
            self._flushes.append((msg["token"], ev))
        elif op == "stop":
            return False
        return True

    def _report(self) -> None:
        with self._lock:
            pending, self._pending = self._pending, {}
            done, self._done = self._done, []
        for rid, toks in pending.items():
            self.outbox.put({"op": "tokens", "id": rid, "tokens": toks})
        for req in done:
            self.live.pop(req.id, None)
            self.outbox.put({"op": "finish", "id": req.id, **{f: getattr(req, f) for f in _RESULT_FIELDS}})
        for token, ev in [f for f in self._flushes if f[1].done.is_set()]:
            self.outbox.put({"op": "flushed", "token": token, "result": dict(ev.result)})
        self._flushes = [f for f in self._flushes if not f[1].done.is_set()]

    def _metrics(self) -> dict:
        kv = self.sched.engine.kv
        return {"op": "metrics", "metrics": asdict(self.sched.metrics),
                "kv": {"num_pages": kv.num_pages, "free_pages": kv.free_pages, "tokens_per_page": kv.tokens_per_page}}

    def _run(self) -> None:
        last_metrics = 0.0
        running = True
        while running and not self._stop.is_set():
            for msg in self.inbox.drain():
                running = self._handle(msg) and running
            self._report()
            if time.time() - last_metrics >= self.metrics_every_s:
                self.outbox.put(self._metrics())
                last_metrics = time.time()
            self._wake.wait(self.poll_s)                         # tokens are reported as they appear, commands within poll_s
            self._wake.clear()
        self._report()


class ReplicaProxy:
    """The front end's handle on a remote replica: same calls as a scheduler, carried over the mailboxes."""

    def __init__(self, store, replica: int, poll_s: float = 0.005):
        self.replica = replica
        self.inbox, self.outbox = Mailbox(store, f"dp/{replica}/in"), Mailbox(store, f"dp/{replica}/out")
        self.poll_s = poll_s
        self.live: Dict[str, GenerationRequest] = {}
        self.metrics = ServerMetrics()
        self.engine = SimpleNamespace(kv=SimpleNamespace(num_pages=0, free_pages=0, tokens_per_page=64))
        self._flushes: Dict[int, CacheFlushEvent] = {}
        self._next_flush = 0
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def start(self) -> "ReplicaProxy":
        self._thread = threading.Thread(target=self._run, name=f"dp-proxy-{self.replica}", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self.inbox.put({"op": "stop"})
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)

    def submit(self, req: GenerationRequest) -> None:
        with self._lock:
            self.live[req.id] = req
        self.inbox.put(_wire_request(req))

    def _flush(self, kind: str) -> CacheFlushEvent:
        ev = CacheFlushEvent(kind)
        with self._lock:
            token = self._next_flush
            self._next_flush += 1
            self._flushes[token] = ev
        self.inbox.put({"op": "flush", "kind": kind, "token": token})
        return ev

    def flush_gpu_cache(self) -> CacheFlushEvent:
        return self._flush("flush_gpu_cache")

    def flush_host_cache(self) -> CacheFlushEvent:
        return self._flush("flush_host_cache")

    def _apply(self, msg: dict) -> None:
        op = msg["op"]
        if op == "tokens":
            req = self.live.get(msg["id"])
            if req is None:
                return
            for t in msg["tokens"]:
                if req.first_token_at is None:
                    req.first_token_at = time.time()
                req.generated.append(t)
                if req.on_token is not None:
                    req.on_token(t)
        elif op == "finish":
            with self._lock:
                req = self.live.pop(msg["id"], None)
            if req is None:
                return
            for f in _RESULT_FIELDS:
                setattr(req, f, msg[f])
            if req.on_finish is not None:
                req.on_finish(req)
        elif op == "flushed":
            with self._lock:
                ev = self._flushes.pop(msg["token"], None)
            if ev is not None:
                ev.result.update(msg["result"])
                ev.done.set()
        elif op == "metrics":
            known = {f.name for f in fields(ServerMetrics)}
            self.metrics = ServerMetrics(**{k: v for k, v in msg["metrics"].items() if k in known})
            self.engine.kv = SimpleNamespace(**msg["kv"])

    def _run(self) -> None:
        while not self._stop.is_set():
            for msg in self.outbox.drain():
                self._apply(msg)
            with self._lock:
                gone = [r for r in self.live.values() if r.cancelled and not r.cancel_seen]
            for r in gone:                                       # the client went away: tell the replica once
                r.cancel_seen = True
                self.inbox.put({"op": "cancel", "id": r.id})
            self.outbox.wait_next(max(self.poll_s, 0.02))        # wakes as soon as the replica stores its next message


class DataParallelRouter:
    """What the front end sees instead of one scheduler: `replicas[0]` is normally the local `GenerationScheduler`,
    the others are `ReplicaProxy` objects."""

    AFFINITY_SLACK = 2            # a prefix-affine replica may hold this many more live requests than the idlest one

    def __init__(self, replicas: List[object], page_tokens: int = 64, max_affinity_entries: int = 65536):
        assert replicas
        self.replicas = replicas
        self.page_tokens = page_tokens
        self.load = [0] * len(replicas)
        self.routed = [0] * len(replicas)
        self._affinity: Dict[int, int] = {}
        self._max_aff = max_affinity_entries
        self._lock = threading.Lock()
        self.engine = SimpleNamespace(kv=_AggregateKv(replicas))

    def choose(self, input_ids) -> int:
        """Replica for a prompt (call with the lock held)."""
        idlest = min(range(len(self.replicas)), key=lambda i: (self.load[i], i))
        if len(input_ids) > self.page_tokens:                    # shorter prompts share no whole KV page
            key = hash(tuple(input_ids[:self.page_tokens]))
            seen = self._affinity.get(key)
            if seen is not None and self.load[seen] <= self.load[idlest] + self.AFFINITY_SLACK:
                return seen
            if len(self._affinity) >= self._max_aff:
                self._affinity.clear()
            self._affinity[key] = idlest
        return idlest

    def submit(self, req: GenerationRequest) -> None:
        with self._lock:
            i = self.choose(req.input_ids)
            self.load[i] += 1
            self.routed[i] += 1
        user_finish = req.on_finish

        def finished(r, i=i):
            with self._lock:
                self.load[i] -= 1
            if user_finish is not None:
                user_finish(r)
        req.on_finish = finished
        self.replicas[i].submit(req)

    def _flush(self, kind: str) -> CacheFlushEvent:
        parts = [getattr(r, kind)() for r in self.replicas]
        total = CacheFlushEvent(kind)

        def wait_all():
            for p in parts:
                p.done.wait(timeout=60)
                for k, v in p.result.items():
                    total.result[k] = total.result.get(k, 0) + v
            total.done.set()
        threading.Thread(target=wait_all, name="dp-flush", daemon=True).start()
        return total

    def flush_gpu_cache(self) -> CacheFlushEvent:
        return self._flush("flush_gpu_cache")

    def flush_host_cache(self) -> CacheFlushEvent:
        return self._flush("flush_host_cache")

    @property
    def metrics(self) -> ServerMetrics:
        """Sum of the replicas' counters (remote replicas: their latest snapshot)."""
        total = ServerMetrics()
        for r in self.replicas:
            m = r.metrics
            for f in fields(ServerMetrics):
                v = getattr(m, f.name)
                if isinstance(v, dict):
                    acc = getattr(total, f.name)
                    for k, x in v.items():
                        acc[k] = acc.get(k, 0) + x
                else:
                    setattr(total, f.name, getattr(total, f.name) + v)
        return total


class _AggregateKv:
    """KV page gauges over all replicas for `/metrics`."""

    def __init__(self, replicas):
        self._replicas = replicas

    @property
    def num_pages(self) -> int:
        return sum(r.engine.kv.num_pages for r in self._replicas)

    @property
    def free_pages(self) -> int:
        return sum(r.engine.kv.free_pages for r in self._replicas)

    @property
    def tokens_per_page(self) -> int:
        return self._replicas[0].engine.kv.tokens_per_page
