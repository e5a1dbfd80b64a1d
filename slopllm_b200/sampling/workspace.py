"""Device-resident sampling state: per-row parameter banks, penalty history, counter RNG.

Parity: `src/sampling.ts:25-431` (`SamplingWorkspace`: sample / sampleDraft / prepareVerification /
verify -> specRejectLinear; capacity 256 rows) over the kernels of `csrc/glm_sampling.cu`.
On CPU (reference op set) the same interface runs the PyTorch definitions from
`slopllm_b200.ops.reference`, using the identical counter RNG, so CPU and GPU draw the same
tokens from the same logits.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from ..config import SamplingParams
from ..ops import reference as R

MAX_ROWS = 256
MAX_CAND = 256        # candidate-set capacity per row (reference: `src/sampling.ts:25-64`)


class SamplingWorkspace:
    def __init__(self, device, vocab_size: int, window: int = 64, max_k: int = MAX_CAND, seed: int = 0):
        self.device = torch.device(device)
        self.vocab = vocab_size
        self.window = window
        self.max_k = min(max_k, MAX_CAND)
        d = self.device
        self.temperature = torch.zeros(MAX_ROWS, dtype=torch.float32, device=d)
        self.top_p = torch.ones(MAX_ROWS, dtype=torch.float32, device=d)
        self.top_k = torch.zeros(MAX_ROWS, dtype=torch.int32, device=d)
        self.rep = torch.ones(MAX_ROWS, dtype=torch.float32, device=d)
        self.presence = torch.zeros(MAX_ROWS, dtype=torch.float32, device=d)
        self.history = torch.full((MAX_ROWS, window), -1, dtype=torch.int64, device=d)
        self.hist_len = torch.zeros(MAX_ROWS, dtype=torch.int32, device=d)
        self.counter = torch.tensor([seed & 0xFFFFFFFF], dtype=torch.int64 if d.type == "cpu" else torch.int32, device=d)
        self.rows: List[Optional[SamplingParams]] = [None] * MAX_ROWS
        self._rows_cache = {}

    def rows_tensor(self, rows: Sequence[int]) -> torch.Tensor:
        """Row-index tensor, cached so that CUDA-graph capture never needs a host copy."""
        key = tuple(rows)
        t = self._rows_cache.get(key)
        if t is None:
            t = torch.as_tensor(list(rows), dtype=torch.int64, device=self.device)
            self._rows_cache[key] = t
        return t

    # ---- row management -------------------------------------------------------------------------
    def set_row(self, row: int, params: SamplingParams, history: Sequence[int] = ()) -> None:
        self.rows[row] = params
        self.temperature[row] = 0.0 if params.greedy else params.temperature
        self.top_p[row] = params.top_p
        self.top_k[row] = params.top_k
        self.rep[row] = params.repetition_penalty
        self.presence[row] = params.presence_penalty
        h = list(history)[-self.window:]
        self.history[row].fill_(-1)
        if h:
            self.history[row, : len(h)] = torch.as_tensor(h, dtype=torch.int64)
        self.hist_len[row] = len(h)

    def all_greedy(self, rows: Sequence[int]) -> bool:
        return all(self.rows[r] is None or self.rows[r].greedy for r in rows)

    def uses_penalties(self, rows: Sequence[int]) -> bool:
        return any(self.rows[r] is not None and (self.rows[r].repetition_penalty != 1.0 or self.rows[r].presence_penalty != 0.0)
                   for r in rows)

    def record(self, rows: Sequence[int], tokens: Sequence[int]) -> None:
        """Append the sampled tokens to the rows' penalty windows (ring of the last `window`)."""
        for r, t in zip(rows, tokens):
            n = int(self.hist_len[r])
            if n < self.window:
                self.history[r, n] = t
                self.hist_len[r] = n + 1
            else:
                self.history[r] = torch.roll(self.history[r], -1)
                self.history[r, -1] = t

    # ---- sampling ----------------------------------------------------------------------------------
    def _gather(self, t: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        return t.index_select(0, rows)

    def sample(self, logits: torch.Tensor, rows: Sequence[int], stream: int = 0, want_candidates: bool = False,
               advance: bool = True):
        """logits [B, V] (fp32) for the given workspace rows -> tokens int64 [B]
        (+ candidate ids / probs [B, max_k] when requested)."""
        B = logits.shape[0]
        rows_t = self.rows_tensor(rows)
        if self.device.type == "cuda":
            out = self._sample_cuda(logits, rows_t, stream, want_candidates)
        else:
            out = self._sample_ref(logits, rows_t, stream, want_candidates)
        if advance:
            self.advance(B)
        return out

    def advance(self, n: int) -> None:
        if self.device.type == "cuda":
            from ..ops import native as N
            N.call("sl_advance_counter", self.counter.data_ptr(), n, N.stream())
        else:
            self.counter[0] = (int(self.counter[0]) + n) & 0xFFFFFFFF

    def _sample_ref(self, logits, rows_t, stream, want_candidates):
        lg = R.apply_penalties(logits, self._gather(self.history, rows_t), self._gather(self.hist_len, rows_t),
                               self._gather(self.rep, rows_t), self._gather(self.presence, rows_t))
        ids, probs = R.sample_distribution(lg, self._gather(self.temperature, rows_t), self._gather(self.top_k, rows_t),
                                           self._gather(self.top_p, rows_t), self.max_k)
        u = R.uniform_from_counter(int(self.counter[0]), rows_t, stream)
        tok = R.sample_from_candidates(ids, probs, u)
        return (tok, ids, probs) if want_candidates else tok

    def _sample_cuda(self, logits, rows_t, stream, want_candidates):
        from ..ops import native as N
        B, V = logits.shape
        lg = logits if logits.dtype == torch.float32 and logits.is_contiguous() else logits.to(torch.float32).contiguous()
        dev = self.device
        g = lambda t: t.index_select(0, rows_t).contiguous()
        temp, top_p, top_k, rep, pres = g(self.temperature), g(self.top_p), g(self.top_k), g(self.rep), g(self.presence)
        hist, hlen = g(self.history), g(self.hist_len)
        rows32 = rows_t.to(torch.int32)
        out = torch.empty(B, dtype=torch.int64, device=dev)
        cid = torch.empty(B, self.max_k, dtype=torch.int64, device=dev) if want_candidates else None
        cpr = torch.empty(B, self.max_k, dtype=torch.float32, device=dev) if want_candidates else None
        p = N.SampleParams(logits=lg.data_ptr(), V=V, ld=lg.stride(0), temperature=temp.data_ptr(), top_p=top_p.data_ptr(),
                           rep_penalty=rep.data_ptr(), presence_penalty=pres.data_ptr(), top_k=top_k.data_ptr(),
                           history=hist.data_ptr(), hist_len=hlen.data_ptr(), window=self.window, max_k=self.max_k,
                           counter=self.counter.data_ptr(), stream=stream, row_ids=rows32.data_ptr(), out_token=out.data_ptr(),
                           cand_ids=N.ptr(cid), cand_probs=N.ptr(cpr))
        N.call("sl_sample", C.byref(p), B, N.stream())
        return (out, cid, cpr) if want_candidates else out

    # ---- speculative verification -----------------------------------------------------------------------
    def verify(self, draft_tokens, draft_ids, draft_probs, target_ids, target_probs):
        """Linear-chain rejection sampling.  Shapes: draft_tokens [B, D]; draft_* [B, D, C];
        target_* [B, D+1, C].  Returns (out_tokens int64 [B, D+1] (-1 padded), num_accepted [B])."""
        B, D = draft_tokens.shape
        Cc = draft_ids.shape[-1]
        if self.device.type != "cuda":
            rows = torch.arange(B)
            cnt = int(self.counter[0])
            ua = torch.stack([R.uniform_from_counter(cnt, rows, 2 * i + 1) for i in range(D)], 1)
            ur = torch.stack([R.uniform_from_counter(cnt, rows, 2 * i + 2) for i in range(D + 1)], 1)
            out = R.spec_reject_linear(draft_tokens, draft_ids, draft_probs, target_ids, target_probs, ua, ur)
            self.advance(B)
            return out
        from ..ops import native as N
        dev = self.device
        out = torch.empty(B, D + 1, dtype=torch.int64, device=dev)
        nacc = torch.empty(B, dtype=torch.int32, device=dev)
        c = lambda t, dt: t.to(dt).contiguous()
        dt_, di, dp = c(draft_tokens, torch.int64), c(draft_ids, torch.int64), c(draft_probs, torch.float32)
        ti, tp = c(target_ids, torch.int64), c(target_probs, torch.float32)
        p = N.SpecRejectParams(draft_tokens=dt_.data_ptr(), draft_ids=di.data_ptr(), draft_probs=dp.data_ptr(),
                               target_ids=ti.data_ptr(), target_probs=tp.data_ptr(), D=D, C=Cc, counter=self.counter.data_ptr(),
                               out_tokens=out.data_ptr(), num_accepted=nacc.data_ptr())
        N.call("sl_spec_reject", C.byref(p), B, N.stream())
        self.advance(B)
        return out, nacc.to(torch.int64)
