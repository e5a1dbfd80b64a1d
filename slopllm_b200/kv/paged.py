"""Paged KV cache bookkeeping: 64-token pages, refcounts, prefix sharing, copy-on-write,
"resume" of a finished conversation, staging of finished sequences, host tier.

Semantics follow the reference (`src/paged_kv.ts:25-531`, `src/paged_sequence.ts:1-160`):

* a sequence owns a list of page ids; whole pages can be shared between sequences by
  refcount; the last partial page of a sequence is private; writing into a shared page
  first copies it (copy-on-write);
* a prefix match never consumes the whole prompt: at most ``floor((len-1)/tokens_per_page)``
  pages are shared, so at least one token is prefilled to produce logits;
* "resume": when a staged donor sequence is an exact proper prefix of the new prompt, is
  fully reported and is the only owner of its last page, the request adopts the donor
  object itself and continues in place (the multi-turn chat fast path);
* finished sequences are staged (pages retained, found by prefix match) until evicted;
* under context parallelism the same page ids are used on every rank and one page covers
  ``64 * W`` consecutive tokens.

The page pool itself (free list + refcounts) lives in the native runtime library
(`csrc/runtime/page_pool.cpp`); this module holds the token-level logic.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence as Seq, Tuple

from ..config import PAGE_SIZE
from ..runtime.native_runtime import PagePool


class PageAllocationError(RuntimeError):
    """Raised when the pool cannot supply the pages a request needs."""


@dataclass
class Sequence:
    seq_id: int
    pages: List[int] = field(default_factory=list)
    token_ids: List[int] = field(default_factory=list)    # every token that has KV allocated
    reported: int = 0                                     # tokens whose KV is known to be written
    shared_prefix_tokens: int = 0                         # tokens adopted from the prefix cache

    @property
    def length(self) -> int:
        return len(self.token_ids)


class PagedKVCache:
    def __init__(self, num_pages: int, cp_world: int = 1, copy_page: Optional[Callable[[int, int], None]] = None):
        self.num_pages = num_pages
        self.tokens_per_page = PAGE_SIZE * cp_world
        self.pool = PagePool(num_pages)
        self.copy_page = copy_page or (lambda src, dst: None)     # device copy of one page in every layer
        self.sequences: Dict[int, Sequence] = {}
        self.staged: Dict[int, Sequence] = {}                     # finished sequences kept for prefix reuse
        self.prefix_sharing = True                                # off for models whose state is not in the pages
        self._next_id = 0

    # ---- pool ----------------------------------------------------------------------------------------
    @property
    def free_pages(self) -> int:
        return self.pool.free_count()

    def _alloc(self, n: int) -> List[int]:
        if n <= 0:
            return []
        pages = self.pool.alloc(n)
        if pages is None:
            raise PageAllocationError(f"need {n} pages, {self.free_pages} free")
        return pages

    def _release(self, pages: Seq[int]) -> None:
        for p in pages:
            self.pool.unref(p)

    def pages_for(self, n_tokens: int) -> int:
        return -(-n_tokens // self.tokens_per_page)

    # ---- sequences ---------------------------------------------------------------------------------------
    def new_sequence(self) -> Sequence:
        s = Sequence(self._next_id)
        self._next_id += 1
        self.sequences[s.seq_id] = s
        return s

    def append_tokens(self, s: Sequence, tokens: Seq[int]) -> None:
        """Reserve KV room for `tokens` at the end of `s` (allocating / un-sharing pages)."""
        new_len = s.length + len(tokens)
        need = self.pages_for(new_len)
        # writing into the current last page: it must be private
        if s.length % self.tokens_per_page != 0 and s.pages:
            self._make_private(s, len(s.pages) - 1)
        if need > len(s.pages):
            s.pages.extend(self._alloc(need - len(s.pages)))
        s.token_ids.extend(int(t) for t in tokens)

    def _make_private(self, s: Sequence, page_index: int) -> None:
        p = s.pages[page_index]
        if self.pool.refcount(p) > 1:
            q = self._alloc(1)[0]
            self.copy_page(p, q)
            self.pool.unref(p)
            s.pages[page_index] = q

    def report_tokens(self, s: Sequence, upto: Optional[int] = None) -> None:
        s.reported = s.length if upto is None else min(upto, s.length)

    def truncate(self, s: Sequence, new_len: int) -> None:
        """Drop tokens (and whole pages that become empty) - MTP over-allocates D+1 tokens
        per step and truncates to committed + accepted + 1."""
        if new_len >= s.length:
            return
        del s.token_ids[new_len:]
        keep = self.pages_for(new_len)
        self._release(s.pages[keep:])
        del s.pages[keep:]
        s.reported = min(s.reported, new_len)

    def free_sequence(self, s: Sequence) -> None:
        self._release(s.pages)
        s.pages = []
        s.token_ids = []
        self.sequences.pop(s.seq_id, None)
        self.staged.pop(s.seq_id, None)

    def stage(self, s: Sequence) -> None:
        """Keep a finished sequence's pages for later prefix matches."""
        self.sequences.pop(s.seq_id, None)
        del s.token_ids[s.reported:]
        keep = self.pages_for(s.reported)
        self._release(s.pages[keep:])
        del s.pages[keep:]
        if s.pages and self.prefix_sharing:
            self.staged[s.seq_id] = s
        elif s.pages:
            self._release(s.pages)
            s.pages = []

    # ---- prefix sharing ----------------------------------------------------------------------------------------
    def match_prefix(self, prompt: Seq[int]) -> Tuple[Optional[Sequence], int, bool]:
        """Best donor among live + staged sequences.  Returns (donor, shared_tokens, resume)."""
        tpp = self.tokens_per_page
        max_pages = (len(prompt) - 1) // tpp if prompt else 0
        best: Tuple[Optional[Sequence], int, bool] = (None, 0, False)
        for cand in list(self.staged.values()) + list(self.sequences.values()):
            n = min(cand.reported, len(prompt))
            m = 0
            ids = cand.token_ids
            while m < n and ids[m] == prompt[m]:
                m += 1
            # resume: donor is an exact proper prefix, staged, sole owner of its last page
            if (cand.seq_id in self.staged and m == cand.reported == cand.length and m < len(prompt)
                    and m % tpp != 0 and cand.pages and self.pool.refcount(cand.pages[-1]) == 1):
                if m > best[1]:
                    best = (cand, m, True)
                continue
            pages = min(m // tpp, max_pages)
            if pages * tpp > best[1]:
                best = (cand, pages * tpp, False)
        return best

    def start_request(self, prompt: Seq[int]) -> Tuple[Sequence, int]:
        """Create (or resume) the sequence for a prompt.  Returns (sequence, cached_tokens):
        KV of the first `cached_tokens` tokens is already present."""
        donor, shared, resume = self.match_prefix(prompt) if self.prefix_sharing else (None, 0, False)
        if donor is not None and resume:
            self.staged.pop(donor.seq_id)
            self.sequences[donor.seq_id] = donor
            donor.shared_prefix_tokens = shared
            return donor, shared
        s = self.new_sequence()
        if donor is not None and shared > 0:
            n = shared // self.tokens_per_page
            for p in donor.pages[:n]:
                self.pool.ref(p)
            s.pages = list(donor.pages[:n])
            s.token_ids = list(prompt[:shared])
            s.reported = shared
            s.shared_prefix_tokens = shared
        return s, shared

    # ---- eviction ---------------------------------------------------------------------------------------------------
    def evict_staged(self, need_pages: int, offload: Optional[Callable[[Sequence], None]] = None) -> int:
        """Free staged sequences, largest first, until `need_pages` are free.  `offload`
        (host tier) sees each victim before its pages are released."""
        freed = 0
        while self.free_pages < need_pages and self.staged:
            victim = max(self.staged.values(), key=lambda s: len(s.pages))
            if offload is not None:
                offload(victim)
            before = self.free_pages
            self.free_sequence(victim)
            freed += self.free_pages - before
        return freed

    def flush_staged(self) -> None:
        for s in list(self.staged.values()):
            self.free_sequence(s)

    def assert_clear(self) -> None:
        assert not self.sequences and not self.staged and self.free_pages == self.num_pages

    # ---- device tables ----------------------------------------------------------------------------------------------
    def page_table_rows(self, seqs: Seq[Sequence], width: int) -> List[List[int]]:
        return [list(s.pages[:width]) + [0] * (width - len(s.pages[:width])) for s in seqs]
