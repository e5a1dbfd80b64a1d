"""Continuous-batching scheduler: admission with prefix reuse (GPU tier, then pinned-host tier),
chunked prefill, batched decode (plain or MTP speculative), per-batch error rollback.

Parity: `src/generation-scheduler.ts:79-338` (`PrefixTierPolicy`) and `:357-692`
(`GenerationScheduler.run`).  One loop iteration = `step()`:

  1. retire finished rows (their sequences are *staged* so later prompts can share / resume them)
  2. drain the event queue: new requests (admitted while rows are free) and cache-flush controls
  3. chunked prefill of admitted prompts under a token budget; a finished prompt yields its
     first token and joins the decode set
  4. one decode step for every row in the decode set
  5. on an exception: every admitted request ends with an error, caches are reset; errors that
     look like a lost CUDA context are re-raised so that the process exits

The engine contract is small (see `EngineLike`) so the scheduler tests run against a fake.
"""
from __future__ import annotations

import queue
import re
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Protocol, Sequence as Seq

from ..config import SamplingParams
from ..kv.paged import PageAllocationError, PagedKVCache, Sequence

_FATAL = re.compile(r"illegal memory access|misaligned address|device-side assert|unspecified launch failure|"
                    r"CUDA context.*destroyed|illegal instruction", re.I)


def is_fatal_cuda_error(err: BaseException) -> bool:
    return bool(_FATAL.search(str(err)))


@dataclass
class GenerationRequest:
    id: str
    input_ids: List[int]
    max_tokens: int = 256
    sampling: SamplingParams = field(default_factory=SamplingParams)
    on_token: Optional[Callable[[int], None]] = None          # called from the scheduler thread
    on_finish: Optional[Callable[["GenerationRequest"], None]] = None
    stop_token_ids: Seq[int] = ()
    # filled in by the scheduler
    generated: List[int] = field(default_factory=list)
    finish_reason: str = ""
    error: Optional[str] = None
    prompt_tokens: int = 0
    cached_tokens: int = 0
    prefill_tokens: int = 0
    prefill_seconds: float = 0.0
    cancelled: bool = False                  # set by the client side at any time
    cancel_reason: str = ""                  # finish reason the row gets when the cancellation is acted on ("" = "cancelled")
    cancel_seen: bool = False                # what the scheduler acts on (copied at step boundaries, on every rank alike)
    retired: bool = False                    # the scheduler has let go of the request (finished, failed or refused)
    submitted_at: float = field(default_factory=time.time)
    first_token_at: Optional[float] = None

    def cancel(self, reason: str = "") -> None:
        """Client side (any thread): the client went away, or it has seen a stop string (`reason="stop"`).  Only this flag
        is written here; the scheduler drops the row, on every rank in the same step, once the cancellation has reached
        all ranks, and assigns `finish_reason` then."""
        if reason and not self.cancel_reason:
            self.cancel_reason = reason
        self.cancelled = True


@dataclass
class CacheFlushEvent:
    kind: str                                    # "flush_gpu_cache" | "flush_host_cache"
    done: threading.Event = field(default_factory=threading.Event)
    result: Dict[str, int] = field(default_factory=dict)


@dataclass
class ServerMetrics:
    running_requests: int = 0
    generation_tokens_total: int = 0
    prompt_tokens_total: int = 0
    cached_prompt_tokens_total: int = 0
    spec_decode_num_drafts_total: int = 0
    spec_decode_num_draft_tokens_total: int = 0
    spec_decode_num_accepted_tokens_total: int = 0
    request_success_total: int = 0
    request_error_total: int = 0
    prefill_time_seconds_count: int = 0
    prefill_time_seconds_sum: float = 0.0
    collective_timeouts_total: int = 0
    rank_failures_total: int = 0
    phase_seconds: Dict[str, float] = field(default_factory=dict)
    phase_count: Dict[str, int] = field(default_factory=dict)

    def record_phase(self, name: str, batch: int, seconds: float) -> None:
        key = f"{name}/b{batch}"
        self.phase_seconds[key] = self.phase_seconds.get(key, 0.0) + seconds
        self.phase_count[key] = self.phase_count.get(key, 0) + 1


class EngineLike(Protocol):
    kv: PagedKVCache
    mtp: int

    def prefill(self, seqs, prompts, chunk_size=..., want_hidden=..., rows=...): ...
    def decode_step(self, seqs, last_tokens, rows=...): ...
    def mtp_seed(self, seqs, last_tokens, last_hiddens): ...
    def mtp_decode_step(self, seqs, last_tokens, seed, rows=...): ...


class HostTier:
    """Pinned-host copy of staged sequences' KV pages (second prefix tier).

    `save(seq)` copies a victim's pages device->host before the GPU tier frees them;
    `match(prompt)` finds the longest page-aligned host prefix; `restore(entry, seq)` copies
    pages host->device into freshly allocated pages of `seq`.  Page copies go through the two
    callbacks so that the tier is independent of the cache tensor layout.
    """

    def __init__(self, max_pages: int, tokens_per_page: int, read_page: Callable[[int], object],
                 write_page: Callable[[int, object], None], read_pages: Optional[Callable] = None,
                 write_pages: Optional[Callable] = None):
        self.max_pages = max_pages
        self.tpp = tokens_per_page
        self.read_page, self.write_page = read_page, write_page
        # batched forms (all pages of a sequence in one copy and one synchronisation); without them: page by page
        self.read_pages = read_pages or (lambda pages: [read_page(p) for p in pages])
        self.write_pages = write_pages or (lambda pages, blobs: [write_page(p, b) for p, b in zip(pages, blobs)])
        self.entries: List[dict] = []            # {"tokens": [...], "pages": [blob, ...]}

    @property
    def used_pages(self) -> int:
        return sum(len(e["pages"]) for e in self.entries)

    def save(self, seq: Sequence) -> None:
        n = seq.reported // self.tpp
        if self.max_pages <= 0 or n == 0 or n > self.max_pages:
            return                            # (a sequence larger than the whole tier must not cost the tier its entries)
        while self.entries and self.used_pages + n > self.max_pages:
            self.entries.remove(max(self.entries, key=lambda e: len(e["pages"])))     # largest victim first
        self.entries.append({"tokens": list(seq.token_ids[: n * self.tpp]), "pages": list(self.read_pages(list(seq.pages[:n])))})

    def match(self, prompt: Seq[int]):
        best, best_pages = None, 0
        limit = (len(prompt) - 1) // self.tpp
        for e in self.entries:
            m = 0
            toks = e["tokens"]
            n = min(len(toks), len(prompt))
            while m < n and toks[m] == prompt[m]:
                m += 1
            pages = min(m // self.tpp, limit, len(e["pages"]))
            if pages > best_pages:
                best, best_pages = e, pages
        return best, best_pages

    def flush(self) -> int:
        n = self.used_pages
        self.entries.clear()
        return n


@dataclass
class _Row:
    req: GenerationRequest
    seq: Sequence
    row: int
    prompt_done: bool = False
    last_token: int = -1
    last_hidden: object = None
    seed: object = None                       # MTP seed hidden of this row ([H] tensor)


class GenerationScheduler:
    ADMIT_LOOKAHEAD_TOKENS = 512      # output tokens whose pages are reserved when a request is admitted

    def __init__(self, engine: EngineLike, max_batch: int = 8, chunk_size: int = 8192, eos_token_ids: Seq[int] = (),
                 host_tier: Optional[HostTier] = None, decode_latency_ms: float = 0.0, replica_channel=None, health=None):
        self.engine = engine
        # rank-failure monitor (utils/health.py): while it reports a lost peer no step is launched (its collectives could
        # never complete) and requests are failed at once instead of queueing behind a dead replica
        self.health = health
        # multi-process serving: rank 0 owns the request queue and broadcasts every step's events so that all
        # ranks admit, cancel and flush in the same step (see scheduler/replicated.py)
        self.replica = replica_channel
        self.max_batch = max_batch
        self.chunk_size = chunk_size
        self.eos = set(eos_token_ids)
        self.host_tier = host_tier
        self.decode_latency = decode_latency_ms / 1e3
        self.events: "queue.Queue" = queue.Queue()
        self.rows: List[_Row] = []
        self.metrics = ServerMetrics()
        self._free_rows = list(range(max_batch))[::-1]
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._was_unhealthy = False

    # ---- public -------------------------------------------------------------------------------------
    def _inbox(self) -> "queue.Queue":
        return self.replica.inbox if self.replica is not None else self.events

    def submit(self, req: GenerationRequest) -> None:
        self._inbox().put(req)

    def flush_gpu_cache(self) -> CacheFlushEvent:
        ev = CacheFlushEvent("flush_gpu_cache")
        self._inbox().put(ev)
        return ev

    def flush_host_cache(self) -> CacheFlushEvent:
        ev = CacheFlushEvent("flush_host_cache")
        self._inbox().put(ev)
        return ev

    def start(self) -> None:
        self._thread = threading.Thread(target=self.run, name="scheduler", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        if self.replica is not None:
            self.replica.inbox.put(None)          # travels to every rank with the next exchange
        else:
            self._stop.set()
            self.events.put(None)
        if self._thread:
            self._thread.join(timeout=30)

    def _fail_unhealthy(self) -> None:
        """A peer is gone: end every admitted and every waiting request with an error, answer pending cache flushes."""
        err = RuntimeError(self.health.state.reason or "a rank of this replica is not responding")
        if self.rows:
            self._fail_all(err)
        for q in ([self.replica.inbox] if self.replica is not None else []) + [self.events]:
            while True:
                try:
                    ev = q.get_nowait()
                except queue.Empty:
                    break
                if ev is None:
                    self._stop.set()
                elif isinstance(ev, CacheFlushEvent):
                    ev.done.set()
                else:
                    ev.error, ev.finish_reason, ev.retired = f"RankFailure: {err}", "error", True
                    self.metrics.request_error_total += 1
                    if ev.on_finish:
                        ev.on_finish(ev)
        self.metrics.running_requests = 0

    def run(self) -> None:
        while not self._stop.is_set():
            if self.health is not None and not self.health.is_healthy():
                if not self._was_unhealthy:
                    self.metrics.rank_failures_total += 1
                self._was_unhealthy = True
                self._fail_unhealthy()
                time.sleep(0.02)
                continue
            self._was_unhealthy = False
            if self.replica is not None:
                self.replica.exchange(self)
                if self._stop.is_set():
                    break
                self.step()
                continue
            if not self.rows and self.events.empty():
                ev = self.events.get()
                if ev is None:
                    break
                self.events.put(ev)               # re-queue; step() drains in order
                continue                          # (the wait may have been long: look at the health monitor first)
            self.step()

    # ---- one iteration ----------------------------------------------------------------------------------
    def step(self) -> None:
        try:
            if self.replica is None:
                for r in self.rows:
                    r.req.cancel_seen = r.req.cancel_seen or r.req.cancelled
            self._retire()
            self._drain_events()
            self._prefill()
            self._decode()
        except Exception as err:  # noqa: BLE001
            self._fail_all(err)
            if is_fatal_cuda_error(err):
                raise
        self.metrics.running_requests = len(self.rows)

    def idle(self) -> bool:
        return not self.rows and self.events.empty()

    # ---- phases ---------------------------------------------------------------------------------------------
    def _retire(self) -> None:
        keep = []
        for r in self.rows:
            req = r.req
            done = bool(req.finish_reason) or req.cancel_seen
            if not done:
                keep.append(r)
                continue
            if req.cancel_seen and not req.finish_reason:
                req.finish_reason = req.cancel_reason or "cancelled"
            req.retired = True
            self.engine.kv.stage(r.seq)           # keep the pages for prefix reuse
            self._free_rows.append(r.row)
            if req.finish_reason in ("stop", "length"):
                self.metrics.request_success_total += 1
            if req.on_finish:
                req.on_finish(req)
        self.rows = keep

    def _drain_events(self) -> None:
        while len(self.rows) < self.max_batch or not self.events.empty():
            try:
                ev = self.events.get_nowait()
            except queue.Empty:
                return
            if ev is None:
                self._stop.set()
                return
            if isinstance(ev, CacheFlushEvent):
                self._flush(ev)
                continue
            if len(self.rows) >= self.max_batch:
                # no free row: put it back at the front of a fresh queue, keeping order
                rest = [ev]
                while True:
                    try:
                        rest.append(self.events.get_nowait())
                    except queue.Empty:
                        break
                for e in rest:
                    self.events.put(e)
                return
            self._admit(ev)

    def _flush(self, ev: CacheFlushEvent) -> None:
        kv = self.engine.kv
        if ev.kind == "flush_gpu_cache":
            before = kv.free_pages
            if self.host_tier is not None:
                for s in list(kv.staged.values()):
                    self.host_tier.save(s)
            kv.flush_staged()
            ev.result = {"gpu_pages_freed": kv.free_pages - before,
                         "host_pages_used": self.host_tier.used_pages if self.host_tier else 0}
        else:
            ev.result = {"host_pages_freed": self.host_tier.flush() if self.host_tier else 0}
        ev.done.set()

    def _admit(self, req: GenerationRequest) -> None:
        kv = self.engine.kv
        prompt = req.input_ids
        req.prompt_tokens = len(prompt)
        if not prompt:
            req.error, req.finish_reason, req.retired = "empty prompt", "error", True
            if req.on_finish:
                req.on_finish(req)
            return
        # pages reserved at admission: the prompt plus a bounded look-ahead of output (a request may ask for tens of
        # thousands of tokens and stop after ten; its later pages are found step by step, see `_make_room`)
        need = kv.pages_for(len(prompt) + min(req.max_tokens, self.ADMIT_LOOKAHEAD_TOKENS) + self.engine.mtp + 1)
        offload = self.host_tier.save if self.host_tier else None
        seq = None
        try:
            seq, cached = kv.start_request(prompt)
            resumed = cached % kv.tokens_per_page != 0        # a staged sequence continues in its own partial last page
            # host tier: a longer prefix there is restored into fresh pages (not behind a resumed partial page, whose
            # tokens the host pages would not line up with)
            if self.host_tier is not None and not resumed and cached < len(prompt) - 1:
                entry, pages = self.host_tier.match(prompt)
                if entry is not None and pages * kv.tokens_per_page > cached:
                    extra = pages - len(seq.pages)
                    if kv.free_pages < extra:
                        kv.evict_staged(extra, offload=offload)
                    if kv.free_pages >= extra:
                        self._restore_from_host(seq, entry, pages, prompt)
                        cached = seq.length
            missing = max(0, need - len(seq.pages))
            if kv.free_pages < missing:
                kv.evict_staged(missing, offload=offload)
            if kv.free_pages < kv.pages_for(len(prompt)) - len(seq.pages):
                raise PageAllocationError(f"prompt of {len(prompt)} tokens does not fit in the KV cache")
        except PageAllocationError as err:
            if seq is not None:
                kv.free_sequence(seq)                         # gives back the shared pages it had taken a reference on
            req.error, req.finish_reason, req.retired = str(err), "error", True
            self.metrics.request_error_total += 1
            if req.on_finish:
                req.on_finish(req)
            return
        req.cached_tokens = cached
        self.metrics.prompt_tokens_total += len(prompt)
        self.metrics.cached_prompt_tokens_total += cached
        row = self._free_rows.pop()
        sampler = getattr(self.engine, "sampler", None)
        if sampler is not None:
            sampler.set_row(row, req.sampling, prompt)
        self.rows.append(_Row(req, seq, row))

    def _restore_from_host(self, seq: Sequence, entry: dict, pages: int, prompt) -> None:
        kv = self.engine.kv
        have = len(seq.pages)
        if pages <= have:
            return
        new_pages = kv._alloc(pages - have)
        self.host_tier.write_pages(new_pages, entry["pages"][have:pages])
        seq.pages.extend(new_pages)
        seq.token_ids = list(prompt[: pages * kv.tokens_per_page])
        seq.reported = len(seq.token_ids)
        seq.shared_prefix_tokens = seq.reported

    def _prefill(self) -> None:
        """One prefill call per step: the rows whose prompts are not cached yet share the step's token budget, in
        admission order, and the engine packs their chunks into one forward pass where they fit (a long prompt fills the
        budget alone and continues next step)."""
        budget = self.chunk_size
        todo = []
        for r in self.rows:
            if r.prompt_done or budget <= 0:
                continue
            take = min(len(r.req.input_ids) - r.seq.length, budget)
            if take <= 0:
                continue
            todo.append((r, take, r.seq.length + take))
            budget -= take
        if not todo:
            return
        t0 = time.time()
        toks, hid = self.engine.prefill([r.seq for r, _, _ in todo], [r.req.input_ids for r, _, _ in todo],
                                        chunk_size=self.chunk_size, want_hidden=self.engine.mtp > 0,
                                        rows=[r.row for r, _, _ in todo], limits=[upto for _, _, upto in todo])
        dt = time.time() - t0
        self.metrics.record_phase("prefill", len(todo), dt)
        total = sum(take for _, take, _ in todo)
        for i, (r, take, upto) in enumerate(todo):
            req = r.req
            req.prefill_tokens += take
            req.prefill_seconds += dt * take / max(1, total)
            if upto == len(req.input_ids):
                r.prompt_done = True
                r.last_token = toks[i]
                r.last_hidden = hid[i] if hid else None
                self.metrics.prefill_time_seconds_count += 1
                self.metrics.prefill_time_seconds_sum += req.prefill_seconds
                req.first_token_at = time.time()
                self._publish(r, [toks[i]])

    def _decode(self) -> None:
        active = [r for r in self.rows if r.prompt_done and not r.req.finish_reason and not r.req.cancel_seen]
        if not active:
            return
        if self.decode_latency:
            time.sleep(self.decode_latency)
        seqs = [r.seq for r in active]
        last = [r.last_token for r in active]
        rows = [r.row for r in active]
        self._make_room(seqs)
        t0 = time.time()
        if self.engine.mtp > 0:
            import torch
            for r in active:                      # rows fresh from prefill get their seed once
                if r.seed is None:
                    r.seed = self.engine.mtp_seed([r.seq], [r.last_token], [self._hidden_for(r)])[0]
            seed = torch.stack([r.seed for r in active])
            accepted, new_last, new_seed = self.engine.mtp_decode_step(seqs, last, seed, rows=rows)
            self.metrics.record_phase("mtp_decode", len(active), time.time() - t0)
            for i, r in enumerate(active):
                r.seed = new_seed[i].clone()
            for r, toks, nl in zip(active, accepted, new_last):
                self.metrics.spec_decode_num_drafts_total += 1
                self.metrics.spec_decode_num_draft_tokens_total += self.engine.mtp
                self.metrics.spec_decode_num_accepted_tokens_total += len(toks) - 1
                r.last_token = nl
                r.last_hidden = None
                self._publish(r, toks)
        else:
            new = self.engine.decode_step(seqs, last, rows=rows)
            self.metrics.record_phase("decode", len(active), time.time() - t0)
            for r, t in zip(active, new):
                r.last_token = t
                self._publish(r, [t])

    def _make_room(self, seqs) -> None:
        """Pages the next step will take beyond what the rows hold: found among the staged sequences (largest first, saved
        to the host tier) before the step, so that a long generation grows past its admission reserve."""
        kv = self.engine.kv
        grow = sum(max(0, kv.pages_for(s.length + self.engine.mtp + 2) - len(s.pages)) for s in seqs)
        if grow and kv.free_pages < grow:
            kv.evict_staged(grow, offload=self.host_tier.save if self.host_tier else None)

    def _hidden_for(self, r: _Row):
        if r.last_hidden is None:
            raise RuntimeError("MTP reseed needs the hidden state of the row's last position")
        return r.last_hidden

    def _publish(self, r: _Row, tokens: Seq[int]) -> None:
        req = r.req
        for t in tokens:
            if req.finish_reason:
                break
            req.generated.append(int(t))
            self.metrics.generation_tokens_total += 1
            if int(t) in self.eos or int(t) in req.stop_token_ids:
                req.finish_reason = "stop"            # the end-of-sequence token itself is not streamed
                break
            if req.on_token and not req.cancelled:
                req.on_token(int(t))
            if len(req.generated) >= req.max_tokens:
                req.finish_reason = "length"

    def _fail_all(self, err: BaseException) -> None:
        msg = f"{type(err).__name__}: {err}"
        if "CollectiveTimeout" in type(err).__name__:
            self.metrics.collective_timeouts_total += 1
        for r in self.rows:
            r.req.error, r.req.finish_reason, r.req.retired = msg, "error", True
            self.metrics.request_error_total += 1
            if r.req.on_finish:
                r.req.on_finish(r.req)
            self._free_rows.append(r.row)
            try:
                self.engine.kv.free_sequence(r.seq)
            except Exception:  # noqa: BLE001
                pass
        self.rows = []
        try:
            self.engine.kv.flush_staged()
        except Exception:  # noqa: BLE001
            pass
