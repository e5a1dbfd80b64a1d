"""Scheduler, prefix cache and host tier on a fake engine (no model, no GPU).
Mirrors the reference's `tests/test_generation_scheduler.ts`, `test_prefix_cache.ts`,
`test_prefix_resume.ts`."""
import pytest

from slopllm_b200.config import SamplingParams
from slopllm_b200.kv.paged import PageAllocationError, PagedKVCache
from slopllm_b200.scheduler.scheduler import GenerationRequest, GenerationScheduler, HostTier


class FakeEngine:
    """Allocates pages like the real engine and 'generates' token = (last + 1) % 1000."""

    def __init__(self, pages=32, mtp=0, fail_on=None):
        self.kv = PagedKVCache(pages)
        self.mtp = mtp
        self.prefill_calls = []
        self.decode_batches = []
        self.fail_on = fail_on

    def prefill(self, seqs, prompts, chunk_size=8192, want_hidden=False, rows=None, limits=None):
        toks = []
        for b, (s, p) in enumerate(zip(seqs, prompts)):
            upto = len(p) if limits is None else limits[b]
            self.prefill_calls.append((s.seq_id, s.length, upto))
            self.kv.append_tokens(s, p[s.length:upto])
            self.kv.report_tokens(s)
            toks.append((p[-1] + 1) % 1000 if upto == len(p) else -1)
        return toks, ([None] * len(seqs) if want_hidden else None)

    def decode_step(self, seqs, last, rows=None):
        if self.fail_on is not None and len(self.decode_batches) == self.fail_on:
            self.decode_batches.append(None)
            raise RuntimeError("boom")
        self.decode_batches.append(len(seqs))
        for s, t in zip(seqs, last):
            self.kv.append_tokens(s, [t])
            self.kv.report_tokens(s)
        return [(t + 1) % 1000 for t in last]


def _req(i, prompt, n=4, **kw):
    got = []
    r = GenerationRequest(id=str(i), input_ids=list(prompt), max_tokens=n, sampling=SamplingParams(temperature=0),
                          on_token=got.append, **kw)
    r.got = got
    return r


def _drain(s, limit=200):
    for _ in range(limit):
        if s.idle():
            s.step()       # retire
            return
        s.step()
    raise AssertionError("scheduler did not finish")


def test_continuous_batching_and_finish_reasons():
    eng = FakeEngine()
    s = GenerationScheduler(eng, max_batch=2, chunk_size=64, eos_token_ids=[7])
    reqs = [_req(0, range(10, 20), 5), _req(1, [3, 4], 10), _req(2, range(100, 130), 3)]
    for r in reqs:
        s.submit(r)
    _drain(s)
    assert reqs[0].generated == [20, 21, 22, 23, 24] and reqs[0].finish_reason == "length"
    assert reqs[1].generated == [5, 6, 7] and reqs[1].finish_reason == "stop"          # hit eos
    assert reqs[2].generated == [130, 131, 132]
    assert max(b for b in eng.decode_batches if b) == 2                                   # two rows decoded together
    assert s.metrics.request_success_total == 3 and s.metrics.generation_tokens_total == 11
    assert reqs[0].got == reqs[0].generated


def test_chunked_prefill_budget():
    eng = FakeEngine(pages=64)
    s = GenerationScheduler(eng, max_batch=2, chunk_size=100)
    r = _req(0, range(250), 2)
    s.submit(r)
    _drain(s)
    spans = [(a, b) for (_, a, b) in eng.prefill_calls]
    assert spans == [(0, 100), (100, 200), (200, 250)]
    assert r.generated == [250, 251]


def test_prefix_sharing_resume_and_cow():
    kv = PagedKVCache(16)
    a, cached = kv.start_request(list(range(200)))
    assert cached == 0
    kv.append_tokens(a, list(range(200)))
    kv.report_tokens(a)
    kv.stage(a)
    # shares whole pages only, and never the whole prompt
    b, cached = kv.start_request(list(range(128)) + [999] * 10)
    assert cached == 128 and b.pages == a.pages[:2] and kv.pool.refcount(a.pages[0]) == 2
    c, cached = kv.start_request(list(range(128)))
    assert cached == 64                      # (len - 1) // 64 pages
    # resume: exact proper prefix ending mid-page, donor adopted in place
    d, cached = kv.start_request(list(range(200)) + [5, 6])
    assert d is a and cached == 200
    # appending to the resumed sequence writes into its private last page; shared pages untouched
    kv.append_tokens(d, [5, 6])
    assert d.pages[:2] == b.pages[:2]
    # copy-on-write: b appends into a fresh private page after its 2 shared ones
    kv.append_tokens(b, [999] * 10)
    assert len(b.pages) == 3 and b.pages[2] not in a.pages


def test_truncate_returns_pages_and_allocation_error():
    kv = PagedKVCache(4)
    s = kv.new_sequence()
    kv.append_tokens(s, [1] * 130)
    assert len(s.pages) == 3
    kv.truncate(s, 64)
    assert len(s.pages) == 1 and kv.free_pages == 3
    with pytest.raises(PageAllocationError):
        kv.append_tokens(s, [1] * 400)
    kv.free_sequence(s)
    kv.assert_clear()


def test_eviction_to_host_tier_and_restore():
    eng = FakeEngine(pages=8)
    store = {}
    host = HostTier(16, 64, read_page=lambda p: ("blob", p), write_page=lambda p, blob: store.__setitem__(p, blob))
    s = GenerationScheduler(eng, max_batch=1, chunk_size=512, host_tier=host)
    r1 = _req(0, range(300), 2)
    s.submit(r1)
    _drain(s)
    assert eng.kv.staged                      # finished sequence staged on the GPU tier
    r2 = _req(1, range(1000, 1400), 2)        # needs 7 pages: evicts the staged one, offloading it to the host
    s.submit(r2)
    _drain(s)
    assert host.used_pages == 4
    ev = s.flush_gpu_cache()
    s.step()
    assert ev.done.is_set() and not eng.kv.staged
    r3 = _req(2, list(range(300)) + [1, 2, 3], 2)
    s.submit(r3)
    _drain(s)
    assert r3.cached_tokens == 256 and len(store) == 4      # restored from pinned host pages
    ev = s.flush_host_cache()
    s.step()
    assert ev.result["host_pages_freed"] >= 4


def test_error_rolls_back_the_batch_and_scheduler_survives():
    eng = FakeEngine(fail_on=1)
    s = GenerationScheduler(eng, max_batch=2, chunk_size=64)
    a, b = _req(0, [1, 2, 3], 8), _req(1, [4, 5], 8)
    s.submit(a)
    s.submit(b)
    _drain(s)
    assert a.finish_reason == "error" and "boom" in a.error and b.finish_reason == "error"
    eng.kv.assert_clear()
    c = _req(2, [9], 3)
    s.submit(c)
    _drain(s)
    assert c.generated == [10, 11, 12]


def test_cancel_and_too_long_prompt():
    eng = FakeEngine(pages=2)
    s = GenerationScheduler(eng, max_batch=1, chunk_size=64)
    big = _req(0, range(500), 2)
    s.submit(big)
    s.step()
    assert big.finish_reason == "error" and "fit" in big.error
    r = _req(1, [1], 100)
    s.submit(r)
    s.step()
    r.cancel()
    _drain(s)
    assert r.finish_reason == "cancelled" and len(r.generated) < 100


def test_sequence_page_edges_truncate_and_copy_on_write():
    """Page-edge cases of the KV bookkeeping (reference `tests/test_report_tokens.ts`, `test_sequence_truncate.ts`):
    speculative over-allocation across a page edge and its truncation, re-growing afterwards, truncation into a page
    that is shared with a donor (the next write must un-share it), and reporting never exceeding what is allocated."""
    copies = []
    kv = PagedKVCache(8, copy_page=lambda a, b: copies.append((a, b)))
    tpp = kv.tokens_per_page
    s = kv.new_sequence()
    kv.append_tokens(s, range(tpp - 1))                    # one token short of the page edge
    kv.report_tokens(s)
    assert len(s.pages) == 1 and s.reported == tpp - 1
    kv.append_tokens(s, [7, 8, 9, 10])                     # a speculative step reserves 4 positions across the edge
    assert len(s.pages) == 2 and s.length == tpp + 3 and s.reported == tpp - 1
    kv.report_tokens(s, upto=10 ** 9)                      # never beyond the allocation
    assert s.reported == s.length
    free_before = kv.free_pages
    kv.truncate(s, tpp)                                    # two drafts accepted: exactly fills page 0, page 1 goes back
    assert len(s.pages) == 1 and s.length == s.reported == tpp and kv.free_pages == free_before + 1
    kv.truncate(s, tpp + 5)                                # growing through truncate is a no-op
    assert s.length == tpp
    kv.append_tokens(s, [11])                              # the next token opens a fresh page
    assert len(s.pages) == 2 and s.token_ids[-1] == 11
    kv.report_tokens(s)
    # a second request shares page 0, is cut back into it, and must copy before writing there
    kv.stage(s)
    prompt = list(range(tpp - 1)) + [7] + [500, 501]
    t, cached = kv.start_request(prompt)
    assert cached == tpp and t.pages[0] == s.pages[0] and kv.pool.refcount(t.pages[0]) == 2
    kv.append_tokens(t, prompt[cached:])
    kv.truncate(t, tpp - 10)                               # back inside the shared page
    assert len(t.pages) == 1 and t.pages[0] == s.pages[0] and not copies
    kv.append_tokens(t, [900])
    assert copies == [(s.pages[0], t.pages[0])] and t.pages[0] != s.pages[0] and kv.pool.refcount(s.pages[0]) == 1
    kv.free_sequence(t)
    kv.flush_staged()
    kv.assert_clear()


def test_collective_timeout_rolls_back_and_is_counted():
    """A device wait that expired surfaces as CollectiveTimeout from the step's readback: the batch ends with an error,
    the timeout counter moves and the scheduler keeps serving."""
    from slopllm_b200.ops.native import CollectiveTimeout

    class TimeoutEngine(FakeEngine):
        def decode_step(self, seqs, last, rows=None):
            if len(self.decode_batches) == 1:
                self.decode_batches.append(None)
                raise CollectiveTimeout("device wait on a peer expired at site 3 (expected flag 9, saw 8)")
            return super().decode_step(seqs, last, rows)

    eng = TimeoutEngine()
    s = GenerationScheduler(eng, max_batch=2, chunk_size=64)
    a = _req(0, [1, 2, 3], 8)
    s.submit(a)
    _drain(s)
    assert a.finish_reason == "error" and "CollectiveTimeout" in a.error and a.retired
    assert s.metrics.collective_timeouts_total == 1
    eng.kv.assert_clear()
    b = _req(1, [9], 2)
    s.submit(b)
    _drain(s)
    assert b.generated == [10, 11]


def test_host_restore_evicts_first_and_frees_on_failure():
    """Full pool + a host-tier match: staged sequences are evicted before the host pages are restored; when nothing can
    be evicted the request fails without leaking the pages it shared."""
    eng = FakeEngine(pages=6)
    store = {}
    host = HostTier(16, 64, read_page=lambda p: ("blob", p), write_page=lambda p, blob: store.__setitem__(p, blob))
    s = GenerationScheduler(eng, max_batch=2, chunk_size=512, host_tier=host)
    r1 = _req(0, range(200), 2)                 # 4 pages, staged afterwards
    s.submit(r1)
    _drain(s)
    for sq in list(eng.kv.staged.values()):
        host.save(sq)                           # the host tier holds its 3 whole pages
    eng.kv.flush_staged()
    r2 = _req(1, range(5000, 5300), 2)          # 5 pages of another prompt, staged: the pool is nearly full
    s.submit(r2)
    _drain(s)
    assert eng.kv.free_pages <= 1 and eng.kv.staged
    r3 = _req(2, list(range(200)) + [7, 8], 2)  # host match of 3 pages: needs eviction first
    s.submit(r3)
    _drain(s)
    assert r3.finish_reason == "length" and r3.cached_tokens == 192 and len(store) == 3
    eng.kv.flush_staged()
    eng.kv.assert_clear()
    # nothing to evict and no room: the request is refused and leaves no reference behind
    blocker = eng.kv.new_sequence()
    eng.kv.append_tokens(blocker, [0] * (64 * 5))
    r4 = _req(3, list(range(200)) + [7, 8], 2)
    s.submit(r4)
    s.step()
    assert r4.finish_reason == "error" and r4.retired
    eng.kv.free_sequence(blocker)
    eng.kv.assert_clear()


def test_resumed_partial_page_skips_the_host_tier():
    """A staged sequence that ends mid-page is resumed in place; a longer host-tier match must not be restored behind its
    partial page (the host pages would not line up with the tokens the sequence already holds)."""
    eng = FakeEngine(pages=16)
    writes = []
    host = HostTier(16, 64, read_page=lambda p: ("blob", p), write_page=lambda p, blob: writes.append(p))
    s = GenerationScheduler(eng, max_batch=1, chunk_size=512, host_tier=host)
    long = _req(0, range(300), 1)
    s.submit(long)
    _drain(s)
    for sq in list(eng.kv.staged.values()):
        host.save(sq)                           # 4 whole pages (256 tokens) on the host
    eng.kv.flush_staged()
    short = _req(1, range(100), 1)              # staged with 101 tokens: a partial second page
    s.submit(short)
    _drain(s)
    donor_len = next(iter(eng.kv.staged.values())).reported
    assert donor_len % 64 != 0
    writes.clear()                              # (the short prompt itself restored one whole page from the host)
    r = _req(2, list(range(100)) + [100] + list(range(101, 300)), 1)
    s.submit(r)
    _drain(s)
    assert r.cached_tokens == donor_len and not writes
    assert r.finish_reason == "length"


def test_host_tier_keeps_its_entries_when_a_sequence_is_too_large():
    host = HostTier(2, 64, read_page=lambda p: p, write_page=lambda p, b: None)
    kv = PagedKVCache(16)
    a = kv.new_sequence()
    kv.append_tokens(a, list(range(128)))
    kv.report_tokens(a)
    host.save(a)
    assert host.used_pages == 2
    b = kv.new_sequence()
    kv.append_tokens(b, list(range(1000, 1000 + 64 * 5)))
    kv.report_tokens(b)
    host.save(b)                                # 5 pages > the tier's 2: refused, and a's pages stay
    assert host.used_pages == 2 and host.entries[0]["tokens"][:3] == [0, 1, 2]


def test_admission_reserves_a_bounded_lookahead_and_grows_later():
    """A request with a huge max_tokens must not evict every staged prefix at admission; its pages are found as it grows."""
    eng = FakeEngine(pages=16)
    s = GenerationScheduler(eng, max_batch=1, chunk_size=512)
    first = _req(0, range(300), 1)              # leaves a staged prefix of 5 pages
    s.submit(first)
    _drain(s)
    staged_before = len(eng.kv.staged)
    assert staged_before == 1
    big = _req(1, range(2000, 2010), 65536)     # asks for 64K tokens, 1024 pages: far more than the pool
    s.submit(big)
    s.step()
    assert len(eng.kv.staged) == staged_before and not big.finish_reason       # admitted, nothing evicted yet
    for _ in range(64 * 11):                    # grow past the free pages: the staged prefix goes when it is needed
        s.step()
        if big.finish_reason:
            break
    assert not eng.kv.staged and len(big.generated) > 64 * 10
    big.cancel()
    _drain(s)


def test_one_prefill_call_packs_several_rows_under_the_budget():
    """Three prompts of 30 / 50 / 40 tokens with a chunk budget of 100: the first step prefills 30 + 50 + 20 in one engine
    call, the second the remaining 20 of the third row (the reference's multi-row prefill chunks)."""
    calls = []

    class Packing(FakeEngine):
        def prefill(self, seqs, prompts, chunk_size=8192, want_hidden=False, rows=None, limits=None):
            calls.append([(s.length, lim) for s, lim in zip(seqs, limits)])
            return super().prefill(seqs, prompts, chunk_size, want_hidden, rows, limits)

    eng = Packing(pages=64)
    s = GenerationScheduler(eng, max_batch=4, chunk_size=100)
    reqs = [_req(0, range(30), 2), _req(1, range(100, 150), 2), _req(2, range(200, 240), 2)]
    for r in reqs:
        s.submit(r)
    _drain(s)
    assert calls[0] == [(0, 30), (0, 50), (0, 20)]
    assert calls[1] == [(20, 40)]
    assert [r.generated for r in reqs] == [[30, 31], [150, 151], [240, 241]]
    assert reqs[2].prefill_tokens == 40
