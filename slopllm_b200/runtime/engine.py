"""Execution engine: paged KV + step planning + CUDA-graph decode + MTP speculative decode.

This is the layer the scheduler, the benchmarks and the server call.  It corresponds to the
reference's `ExecutionWorkspace.planDecode/planPrefill` (`src/execution-workspace.ts:553-783`),
`ChatModel.executePrefill/generateDecode` (`src/chat_model.ts:346-449`) and
`Glm51Model.generateMtpDecode` (`src/glm51_model.ts:1195-1469`).

Per decode step the host writes the step's token ids, positions and page table into one
pinned staging buffer, issues a single async H2D copy into the static device buffers the
captured graph reads, replays the graph, and reads the sampled tokens back with one D2H copy.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence as Seq

import torch

from ..config import PAGE_SIZE, GlmMoeDsaConfig
from ..kv.paged import PagedKVCache, Sequence
from ..models.glm_moe_dsa import GlmMoeDsaModel, KVCacheTensors, StepState
from ..ops import reference as R
from ..parallel.dist import ParallelContext
from ..utils.tracing import traced
from .graphs import CaptureManager


STEP_ARENA_BYTES = 16 << 20        # static step inputs / their pinned mirrors and results; larger shapes fall back


@dataclass
class StepBuffers:
    """Static device buffers (+ pinned host mirror) for one (batch, tokens-per-row) shape."""

    B: int
    tpr: int                       # tokens per row in the step (1 decode, D+1 verification)
    width: int                     # page-table width
    host: torch.Tensor             # pinned int32 [n]
    dev: torch.Tensor              # device int32 [n]

    @classmethod
    def create(cls, B: int, tpr: int, width: int, device, host_arena=None, dev_arena=None) -> "StepBuffers":
        """With arenas (`runtime/workspace.py`) the pinned mirror and the device buffer are carved from the engine's two
        step arenas and stay for the engine's life (a captured graph keeps reading the device one); a shape that no
        longer fits gets buffers of its own."""
        n = 3 * B * tpr + B * width
        host = dev = None
        if host_arena is not None and dev_arena is not None:
            try:
                host = host_arena.alloc((n,), torch.int32, name=f"step_host_{B}x{tpr}").zero_()
                dev = dev_arena.alloc((n,), torch.int32, name=f"step_dev_{B}x{tpr}").zero_()
                host_arena.freeze()
                dev_arena.freeze()
            except MemoryError:
                host = dev = None
        if host is None:
            host = torch.zeros(n, dtype=torch.int32, pin_memory=device.type == "cuda")
            dev = torch.zeros(n, dtype=torch.int32, device=device)
        return cls(B, tpr, width, host, dev)

    def views(self, t: torch.Tensor):
        T = self.B * self.tpr
        return t[:T], t[T:2 * T], t[2 * T:3 * T], t[3 * T:].view(self.B, self.width)

    def nbytes(self) -> int:
        return self.host.numel() * 4


class Engine:
    def __init__(self, cfg: GlmMoeDsaConfig, model: GlmMoeDsaModel, num_pages: int, max_batch: int = 8,
                 max_seq_len: int = 16384, cuda_graph: bool = True, mtp: int = 0, sampler=None, phased_prefill: bool = False,
                 phased_min_tokens: int = 2048):
        self.cfg = cfg
        self.model = model
        self.ctx: ParallelContext = model.ctx
        self.device = self.ctx.device
        self.kv = PagedKVCache(num_pages, self.ctx.cp_world, copy_page=self._copy_page)
        self.kv.prefix_sharing = getattr(model, "supports_prefix_sharing", True)
        # model families bring their own cache layout (dense K/V, recurrent state); the flagship uses packed MLA rows
        self.cache = (model.allocate_cache(num_pages) if hasattr(model, "allocate_cache")
                      else KVCacheTensors.allocate(cfg, num_pages, self.device, len(model.w.layers)))
        self.max_batch = max_batch
        self.pt_width = -(-max_seq_len // (PAGE_SIZE * self.ctx.cp_world)) + 1
        self.graphs = CaptureManager(enabled=cuda_graph and self.device.type == "cuda")
        self.mtp = mtp
        self.sampler = sampler               # SamplingWorkspace (row b of a step <-> workspace row rows[b])
        # phased prefill: a chunk of at least `phased_min_tokens` is run as two halves on two streams so that one
        # half's collectives overlap the other half's GEMMs (only useful with more than one rank)
        self.phased_prefill = phased_prefill and hasattr(model, "forward_hidden_phased")
        self.phased_min_tokens = phased_min_tokens
        self._phase_streams = None
        self._bufs = {}
        self._out_host = {}
        # static step inputs (device) and their pinned mirrors + result read-back buffers (host): two small arenas with
        # the reference's explicit workspace model, so a step's host <-> device traffic touches two allocations only
        from .workspace import Workspace
        self.step_arena = Workspace(STEP_ARENA_BYTES, self.device)
        self.host_arena = Workspace(STEP_ARENA_BYTES, "cpu", pinned=self.device.type == "cuda")
        self._err_host = None                # pinned copy of the device's status words, read back with every step result
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    # ---- pages ---------------------------------------------------------------------------------------
    def _copy_page(self, src: int, dst: int) -> None:
        if hasattr(self.cache, "copy_page"):
            self.cache.copy_page(src, dst)
            return
        a, b = slice(src * PAGE_SIZE, (src + 1) * PAGE_SIZE), slice(dst * PAGE_SIZE, (dst + 1) * PAGE_SIZE)
        for lc in self.cache.layers:
            lc.kv[b] = lc.kv[a]
            if lc.idx is not None:
                lc.idx[b] = lc.idx[a]

    # -- page IO for the pinned-host prefix tier (reference `copyPrefixFrom`, `src/paged_kv.ts:308-370`) ---------------
    def _page_tensors(self) -> Optional[List[torch.Tensor]]:
        """The cache tensors whose first dimension is the slot (page * PAGE_SIZE + offset), in a fixed order; None when
        the cache also holds per-sequence state that pages do not capture (recurrent layers)."""
        c = self.cache
        if hasattr(c, "page_tensors"):
            return c.page_tensors()
        out = []
        for lc in c.layers:
            out.append(lc.kv)
            if lc.idx is not None:
                out.append(lc.idx)
        return out

    def supports_host_tier(self) -> bool:
        return self._page_tensors() is not None

    def read_page(self, page: int) -> torch.Tensor:
        """All layers' rows of one page as a single byte buffer on the host (pinned when the cache is on a GPU): the
        layers' slices are packed on the device, so the page crosses PCIe / C2C in one copy."""
        sl = slice(page * PAGE_SIZE, (page + 1) * PAGE_SIZE)
        packed = torch.cat([t[sl].reshape(-1).view(torch.uint8) for t in self._page_tensors()])
        if not packed.is_cuda:
            return packed
        host = torch.empty(packed.numel(), dtype=torch.uint8, pin_memory=True)
        host.copy_(packed, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()        # the blob may be read (or the page reused) right away
        return host

    def read_pages(self, pages: Seq[int]) -> List[torch.Tensor]:
        """`read_page` for many pages with one gather per cache tensor, one device-to-host copy and one synchronisation
        in total (the reference batches its page copies the same way, `src/paged_kv.ts:308-370`)."""
        if not pages:
            return []
        tensors = self._page_tensors()
        idx = torch.as_tensor(list(pages), dtype=torch.int64, device=self.device)
        parts = [t.view(-1, PAGE_SIZE, *t.shape[1:]).index_select(0, idx).reshape(len(pages), -1).view(torch.uint8) for t in tensors]
        packed = torch.cat(parts, dim=1)                                      # [pages, bytes per page]
        if not packed.is_cuda:
            return list(packed.unbind(0))
        host = torch.empty(packed.shape, dtype=torch.uint8, pin_memory=True)
        host.copy_(packed, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return list(host.unbind(0))

    def write_pages(self, pages: Seq[int], blobs: Seq[torch.Tensor]) -> None:
        """Inverse of `read_pages`: one host-to-device copy, one scatter per cache tensor."""
        if not pages:
            return
        tensors = self._page_tensors()
        per_page = sum(t[:PAGE_SIZE].numel() * t.element_size() for t in tensors)
        for b in blobs:
            if b.numel() != per_page:
                raise ValueError(f"page blob of {b.numel()} bytes does not match this cache's page size of {per_page} bytes")
        host = torch.stack([b.reshape(-1) for b in blobs])
        if self.device.type == "cuda" and not host.is_pinned():
            host = host.pin_memory()
        dev = host.to(self.device, non_blocking=True)
        idx = torch.as_tensor(list(pages), dtype=torch.int64, device=self.device)
        off = 0
        for t in tensors:
            n = t[:PAGE_SIZE].numel() * t.element_size()
            rows = dev[:, off:off + n].contiguous().view(t.dtype).reshape(len(pages), PAGE_SIZE, *t.shape[1:])
            t.view(-1, PAGE_SIZE, *t.shape[1:]).index_copy_(0, idx, rows)
            off += n

    def write_page(self, page: int, blob: torch.Tensor) -> None:
        """Inverse of `read_page` into page `page` (one host-to-device copy, then per-layer scatter on the device)."""
        sl = slice(page * PAGE_SIZE, (page + 1) * PAGE_SIZE)
        tensors = self._page_tensors()
        total = sum(t[sl].numel() * t.element_size() for t in tensors)
        if blob.numel() != total:
            raise ValueError(f"page blob of {blob.numel()} bytes does not match this cache's page size of {total} bytes")
        dev = blob.to(self.device, non_blocking=True)
        off = 0
        for t in tensors:
            dst = t[sl]
            n = dst.numel() * dst.element_size()
            dst.copy_(dev[off:off + n].view(t.dtype).reshape(dst.shape))
            off += n

    def _buffers(self, B: int, tpr: int) -> StepBuffers:
        key = (B, tpr)
        if key not in self._bufs:
            self._bufs[key] = StepBuffers.create(B, tpr, self.pt_width, self.device, self.host_arena, self.step_arena)
        return self._bufs[key]

    def _upload(self, buf: StepBuffers, ids, positions, batch_idx, seqs: Seq[Sequence]) -> None:
        h_ids, h_pos, h_bi, h_pt = buf.views(buf.host)
        h_ids[: len(ids)] = torch.as_tensor(ids, dtype=torch.int32)
        h_pos[: len(ids)] = torch.as_tensor(positions, dtype=torch.int32)
        h_bi[: len(ids)] = torch.as_tensor(batch_idx, dtype=torch.int32)
        h_pt.zero_()
        for b, s in enumerate(seqs):
            n = min(len(s.pages), buf.width)
            h_pt[b, :n] = torch.as_tensor(s.pages[:n], dtype=torch.int32)
        buf.dev.copy_(buf.host, non_blocking=True)
        self.h2d_bytes += buf.nbytes()

    def _state(self, buf: StepBuffers, max_kv_len: int, logits_idx=None) -> StepState:
        ids, pos, bi, pt = buf.views(buf.dev)
        return StepState(input_ids=ids, positions=pos, batch_idx=bi, page_table=pt, logits_idx=logits_idx,
                         cp_world=self.ctx.cp_world, cp_rank=self.ctx.cp_rank, max_kv_len=max_kv_len)

    # ---- prefill -------------------------------------------------------------------------------------------
    @traced("prefill")
    def prefill(self, seqs: Seq[Sequence], prompts: Seq[Seq[int]], chunk_size: int = 8192,
                want_hidden: bool = False, rows: Optional[Seq[int]] = None, limits: Optional[Seq[int]] = None):
        """Chunked prefill of each prompt's uncached tail (up to `limits[b]` tokens when given:
        the scheduler spreads a long prompt over several steps).  Returns (next token per
        sequence, last hidden per sequence or None); the token is meaningful only for
        sequences whose whole prompt is now cached.

        Every forward pass takes up to `chunk_size` tokens and packs them from as many sequences as fit, in order: a
        long prompt fills chunks alone, several short tails share one (the reference's `planPrefill(batchSize, lens)`,
        `src/execution-workspace.ts:648-783`, `src/glm51_model.ts:1158-1188`)."""
        B = len(seqs)
        upto = [len(p) if limits is None else min(len(p), limits[b]) for b, p in enumerate(prompts)]
        last_hidden: List[Optional[torch.Tensor]] = [None] * B
        while True:
            spans, budget = [], chunk_size
            for b in range(B):
                start = seqs[b].length
                if start >= upto[b] or budget <= 0:
                    continue
                n = min(budget, upto[b] - start)
                spans.append((b, start, n))
                budget -= n
            if not spans:
                break
            ids: List[int] = []
            positions: List[int] = []
            bidx: List[int] = []
            group = [seqs[b] for b, _, _ in spans]
            for gi, (b, start, n) in enumerate(spans):
                tok = list(prompts[b][start:start + n])
                self.kv.append_tokens(seqs[b], tok)
                ids += tok
                positions += range(start, start + n)
                bidx += [gi] * n
            st = self._eager_state(ids, positions, bidx, group, max_kv_len=max(start + n for _, start, n in spans))
            self._prepare(st, group)
            if len(spans) == 1 and self.phased_prefill and spans[0][2] >= self.phased_min_tokens:
                _, start, n = spans[0]
                hidden = self._forward_phased(ids, positions, group[0], start, n)
            else:
                hidden = self.model.forward_hidden(st, self.cache)
            if self.mtp and getattr(self.cfg, "num_nextn_predict_layers", 0):
                self._prefill_mtp(st, hidden, [(prompts[b], start, n) for b, start, n in spans])
            off = 0
            for b, start, n in spans:
                self.kv.report_tokens(seqs[b])
                last_hidden[b] = hidden[off + n - 1:off + n]
                off += n
        tokens, hiddens = [], []
        for b in range(B):
            if upto[b] < len(prompts[b]) or last_hidden[b] is None:
                tokens.append(-1)
                hiddens.append(last_hidden[b])
                continue
            row = None if rows is None else rows[b]
            if row is not None and self.sampler is not None and not self.sampler.all_greedy([row]):
                tokens.append(int(self._select(last_hidden[b], [row])[0]))
            else:
                tokens.append(int(self._greedy(last_hidden[b])[0]))
            hiddens.append(last_hidden[b])
        self.check_device_errors()           # (the token reads above already synchronised the stream)
        return tokens, (hiddens if want_hidden else None)

    def _forward_phased(self, ids, positions, s: Sequence, start: int, n: int) -> torch.Tensor:
        half = (n // 2 + 63) // 64 * 64
        parts = [(0, half), (half, n)]
        sts = [self._eager_state(ids[a:b], positions[a:b], [0] * (b - a), [s], max_kv_len=start + b) for a, b in parts]
        streams = None
        if self.device.type == "cuda":
            if self._phase_streams is None:
                self._phase_streams = [torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)]
            streams = self._phase_streams
        return torch.cat(self.model.forward_hidden_phased(sts, self.cache, streams), 0)

    def _prefill_mtp(self, st: StepState, hidden, spans) -> None:
        """Fill the MTP layer's KV over the chunk: position i pairs (h_i, token_{i+1}).  `spans` = (prompt, start, n) of
        every sequence packed into the chunk, in order."""
        nxt: List[int] = []
        for prompt, start, n in spans:
            part = list(prompt[start + 1:start + n + 1])
            if len(part) < n:
                part.append(0)       # the pair at the last prompt position is redone at decode time
            nxt += part
        st2 = StepState(input_ids=torch.as_tensor(nxt, dtype=torch.int64, device=self.device), positions=st.positions,
                        batch_idx=st.batch_idx, page_table=st.page_table, cp_world=st.cp_world, cp_rank=st.cp_rank,
                        max_kv_len=st.max_kv_len)
        self.model.forward_mtp(st2, self.cache, hidden)

    def _prepare(self, st: StepState, seqs) -> None:
        """Per-step host work of the model that must stay outside a graph capture (recurrent-state slots)."""
        if hasattr(self.model, "prepare_step"):
            self.model.prepare_step(st, seqs)

    def check_device_errors(self) -> None:
        """Raise if a kernel recorded an expired wait, a failed index self-check or a collective timeout
        since the last call (reads a few status words back from the device)."""
        if self.device.type != "cuda":
            return
        from ..ops import tcgen05
        tcgen05.check_errors(self.device)
        comm = getattr(self.model, "comm", None)
        if comm is not None and hasattr(comm, "check_status"):
            comm.check_status()

    def release(self, s: Sequence) -> None:
        """Tell the model that a sequence is gone (frees per-sequence state outside the page pool)."""
        if hasattr(self.model, "release_sequence"):
            self.model.release_sequence(s.seq_id)

    def _eager_state(self, ids, positions, batch_idx, seqs, max_kv_len, logits_idx=None) -> StepState:
        dev = self.device
        width = max(self.pt_width, max(len(s.pages) for s in seqs))
        pt = torch.tensor(self.kv.page_table_rows(seqs, width), dtype=torch.int32, device=dev)
        st = StepState(input_ids=torch.as_tensor(ids, dtype=torch.int64, device=dev),
                       positions=torch.as_tensor(positions, dtype=torch.int32, device=dev),
                       batch_idx=torch.as_tensor(batch_idx, dtype=torch.int32, device=dev), page_table=pt,
                       logits_idx=logits_idx, cp_world=self.ctx.cp_world, cp_rank=self.ctx.cp_rank,
                       max_kv_len=max_kv_len)
        # rows of one sequence share one page table: the prefill index scorer on the tensor cores takes that case
        st.extra["one_sequence"] = len(batch_idx) > 0 and min(batch_idx) == max(batch_idx)
        return st

    # ---- plain decode -----------------------------------------------------------------------------------------
    @traced("decode_step")
    def decode_step(self, seqs: Seq[Sequence], last_tokens: Seq[int], rows: Optional[Seq[int]] = None) -> List[int]:
        """One token per sequence: append `last_tokens`, run the model, return the next tokens
        (greedy, or drawn by the sampling workspace for its `rows`).  Graph-captured per
        (batch, KV bucket, sampling mode)."""
        B = len(seqs)
        rows = list(range(B)) if rows is None else list(rows)
        sampled = self.sampler is not None and not self.sampler.all_greedy(rows)
        positions = []
        for s, t in zip(seqs, last_tokens):
            positions.append(s.length)
            self.kv.append_tokens(s, [t])
        buf = self._buffers(B, 1)
        self._upload(buf, list(last_tokens), positions, list(range(B)), seqs)
        bucket = R.padded_kv_len(max(positions) + 1)
        st = self._state(buf, bucket)
        self._prepare(st, seqs)

        def run():
            hidden = self.model.forward_hidden(st, self.cache)
            return self._select(hidden, rows if sampled else None)

        out = self.graphs.execute(("decode", B, bucket, tuple(rows) if sampled else None), run)
        host = self._readback(("decode", B), out)
        for s in seqs:
            self.kv.report_tokens(s)
        toks = host.tolist()
        if sampled and self.sampler.uses_penalties(rows):
            self.sampler.record(rows, toks)
        return toks

    def _select(self, hidden: torch.Tensor, rows: Optional[Seq[int]], stream: int = 0) -> torch.Tensor:
        """Next tokens from hidden states: greedy arg-max, or the sampling kernel over the
        full-vocabulary logits for the given workspace rows."""
        if rows is None:
            return self._greedy(hidden)
        logits = self.model.compute_logits(hidden).to(torch.float32)
        return self.sampler.sample(logits, rows, stream=stream)

    def _greedy(self, hidden: torch.Tensor) -> torch.Tensor:
        """Next-token ids from hidden states (vocabulary-sharded lm_head: local argmax, then
        the winner across ranks)."""
        m = self.model
        local = m.ops.logits(hidden, m.w.lm_head)
        if self.ctx.world == 1:
            return m.ops.argmax(local)
        if hasattr(m.ops, "argmax") and self.device.type == "cuda":
            ids, vals = m.ops.argmax(local, id_offset=m.w.vocab_offset, want_val=True)
        else:
            vals, ids = local.max(-1)
            ids = ids + m.w.vocab_offset
        all_v = torch.stack(m.comm.all_gather_list(vals.to(torch.float32)))
        all_i = torch.stack(m.comm.all_gather_list(ids))
        best = all_v.argmax(0, keepdim=True)
        return all_i.gather(0, best).squeeze(0)

    def _readback(self, key, dev_t: torch.Tensor) -> torch.Tensor:
        """Step result device -> pinned host, and with it (same stream, same synchronisation) the device's status words:
        an expired bounded wait of a collective or a persistent kernel, or a failed index self-check, raises here, in the
        step that produced it, so that the scheduler rolls the batch back instead of publishing tokens computed from
        stale data."""
        host = self._out_host.get(key)
        if host is None or host.shape != dev_t.shape or host.dtype != dev_t.dtype:
            try:
                host = self.host_arena.alloc(tuple(dev_t.shape), dev_t.dtype, name=f"result_{key}")
                self.host_arena.freeze()
            except MemoryError:
                host = torch.empty(dev_t.shape, dtype=dev_t.dtype, pin_memory=self.device.type == "cuda")
            self._out_host[key] = host
        host.copy_(dev_t, non_blocking=True)
        if self.device.type == "cuda":
            from ..ops import tcgen05
            if self._err_host is None:
                self._err_host = torch.zeros(tcgen05.ERROR_WORDS, dtype=torch.int32, pin_memory=True)
            self._err_host.copy_(tcgen05.error_flag(self.device), non_blocking=True)
            torch.cuda.current_stream().synchronize()
            self.d2h_bytes += self._err_host.numel() * 4
            if bool(self._err_host.any()):
                tcgen05.raise_for(self._err_host.tolist(), self.device)
        self.d2h_bytes += host.numel() * host.element_size()
        return host

    # ---- MTP speculative decode -----------------------------------------------------------------------------------
    def mtp_seed(self, seqs: Seq[Sequence], last_tokens: Seq[int], last_hiddens: Seq[torch.Tensor]) -> torch.Tensor:
        """After prefill: run the MTP layer at each sequence's last prompt position with the
        pair (h_last, first sampled token).  Returns the seed hidden [B, H] that predicts
        the token after `last_tokens`."""
        B = len(seqs)
        positions = [s.length - 1 for s in seqs]
        st = self._eager_state(list(last_tokens), positions, list(range(B)), seqs, max_kv_len=max(positions) + 1)
        return self.model.forward_mtp(st, self.cache, torch.cat(list(last_hiddens), 0))

    @traced("mtp_decode_step")
    def mtp_decode_step(self, seqs: Seq[Sequence], last_tokens: Seq[int], seed: torch.Tensor,
                        rows: Optional[Seq[int]] = None):
        """One speculative step with D = self.mtp drafts per sequence.  Greedy rows compare
        arg-max tokens; sampled rows draw drafts from the MTP distribution and verify them by
        linear-chain rejection sampling on the device (distribution-preserving).

        Returns (accepted tokens per sequence (1..D+1 each), new last tokens, new seed)."""
        D, B = self.mtp, len(seqs)
        rows = list(range(B)) if rows is None else list(rows)
        sampled = self.sampler is not None and not self.sampler.all_greedy(rows)
        tpr = D + 1
        p0 = [s.length for s in seqs]
        for s, t in zip(seqs, last_tokens):
            self.kv.append_tokens(s, [t] + [0] * D)          # over-allocate D+1, truncated below
        buf = self._buffers(B, tpr)
        ids = []
        positions = []
        bidx = []
        for b in range(B):
            ids += [last_tokens[b]] + [0] * D
            positions += list(range(p0[b], p0[b] + tpr))
            bidx += [b] * tpr
        self._upload(buf, ids, positions, bidx, seqs)
        bucket = R.padded_kv_len(max(positions) + 1)
        st = self._state(buf, bucket)
        seed_buf = self._static("mtp_seed", (B, self.cfg.hidden_size), seed.dtype)
        seed_buf.copy_(seed)

        def run():
            return self._mtp_graph_body(st, seed_buf, B, D, rows if sampled else None)

        out_tokens, n_acc, new_seed = self.graphs.execute(("mtp", B, D, bucket, tuple(rows) if sampled else None), run)
        packed = self._readback(("mtp", B), torch.cat([out_tokens, n_acc.unsqueeze(1)], 1))
        accepted, new_last = [], []
        for b, s in enumerate(seqs):
            a = int(packed[b, tpr])
            toks = [int(x) for x in packed[b, :a + 1]]
            # KV now holds last_token + a accepted drafts; the bonus token is the new last token
            self.kv.truncate(s, p0[b] + a + 1)
            s.token_ids[p0[b] + 1:p0[b] + a + 1] = toks[:a]
            self.kv.report_tokens(s)
            accepted.append(toks)
            new_last.append(toks[-1])
        return accepted, new_last, new_seed

    def _static(self, name: str, shape, dtype) -> torch.Tensor:
        key = (name, tuple(shape), dtype)
        t = self._bufs.get(key)
        if t is None:
            t = torch.zeros(shape, dtype=dtype, device=self.device)
            self._bufs[key] = t
        return t

    def _mtp_graph_body(self, st: StepState, seed: torch.Tensor, B: int, D: int, rows=None):
        if rows is not None:
            return self._mtp_graph_body_sampled(st, seed, B, D, rows)
        m, dev = self.model, self.device
        tpr = D + 1
        ids2d = st.input_ids.view(B, tpr)
        pos2d = st.positions.view(B, tpr)
        rows = torch.arange(B, dtype=torch.int32, device=dev)
        # --- draft chain: d1 from the seed, then D-1 single-token MTP passes ---
        hidden = seed
        for depth in range(D):
            d = self._greedy(hidden)
            ids2d[:, depth + 1] = d.to(ids2d.dtype)
            if depth + 1 < D:
                stp = StepState(input_ids=d, positions=pos2d[:, depth].contiguous(), batch_idx=rows,
                                page_table=st.page_table, cp_world=st.cp_world, cp_rank=st.cp_rank,
                                max_kv_len=st.max_kv_len)
                hidden = m.forward_mtp(stp, self.cache, hidden)
        # --- verification: main model over [last, d1..dD] ---
        h = m.forward_hidden(st, self.cache)
        target = self._greedy(h).view(B, tpr)
        drafts = ids2d[:, 1:].to(target.dtype)
        ok = (drafts == target[:, :D]).to(torch.int32)
        n_acc = torch.cumprod(ok, dim=1).sum(1)                                   # [B]
        j = torch.arange(tpr, device=dev).unsqueeze(0)
        bonus = target.gather(1, n_acc.unsqueeze(1).to(torch.int64))               # [B, 1]
        out_tokens = torch.where(j < n_acc.unsqueeze(1), torch.cat([drafts, drafts[:, :1]], 1), bonus.expand(B, tpr))
        # --- reseed: MTP layer over the verification positions with (h_j, next token_j) ---
        st2 = StepState(input_ids=out_tokens.reshape(-1), positions=st.positions, batch_idx=st.batch_idx,
                        page_table=st.page_table, cp_world=st.cp_world, cp_rank=st.cp_rank, max_kv_len=st.max_kv_len)
        hm = m.forward_mtp(st2, self.cache, h).view(B, tpr, -1)
        new_seed = hm.gather(1, n_acc.view(B, 1, 1).to(torch.int64).expand(B, 1, hm.shape[-1])).squeeze(1)
        return out_tokens, n_acc.to(out_tokens.dtype), new_seed

    def _mtp_graph_body_sampled(self, st: StepState, seed: torch.Tensor, B: int, D: int, rows):
        """Speculative step with sampling: drafts are drawn from the MTP head's candidate
        distribution, the main model's candidate distributions at the D+1 positions verify them."""
        m, dev, sw = self.model, self.device, self.sampler
        tpr = D + 1
        ids2d = st.input_ids.view(B, tpr)
        pos2d = st.positions.view(B, tpr)
        brow = torch.arange(B, dtype=torch.int32, device=dev)
        hidden = seed
        d_tok, d_ids, d_probs = [], [], []
        for depth in range(D):
            logits = m.compute_logits(hidden).to(torch.float32)
            tok, cid, cpr = sw.sample(logits, rows, stream=16 + depth, want_candidates=True, advance=False)
            d_tok.append(tok); d_ids.append(cid); d_probs.append(cpr)
            ids2d[:, depth + 1] = tok.to(ids2d.dtype)
            if depth + 1 < D:
                stp = StepState(input_ids=tok, positions=pos2d[:, depth].contiguous(), batch_idx=brow,
                                page_table=st.page_table, cp_world=st.cp_world, cp_rank=st.cp_rank,
                                max_kv_len=st.max_kv_len)
                hidden = m.forward_mtp(stp, self.cache, hidden)
        h = m.forward_hidden(st, self.cache)
        logits = m.compute_logits(h).to(torch.float32)                               # [B * tpr, V]
        rep_rows = [r for r in rows for _ in range(tpr)]
        _, t_ids, t_probs = sw.sample(logits, rep_rows, stream=48, want_candidates=True, advance=False)
        Cc = t_ids.shape[-1]
        out_tokens, n_acc = sw.verify(torch.stack(d_tok, 1), torch.stack(d_ids, 1), torch.stack(d_probs, 1),
                                      t_ids.view(B, tpr, Cc), t_probs.view(B, tpr, Cc))
        st2 = StepState(input_ids=out_tokens.clamp(min=0).reshape(-1), positions=st.positions, batch_idx=st.batch_idx,
                        page_table=st.page_table, cp_world=st.cp_world, cp_rank=st.cp_rank, max_kv_len=st.max_kv_len)
        hm = m.forward_mtp(st2, self.cache, h).view(B, tpr, -1)
        new_seed = hm.gather(1, n_acc.view(B, 1, 1).to(torch.int64).expand(B, 1, hm.shape[-1])).squeeze(1)
        return out_tokens, n_acc.to(out_tokens.dtype), new_seed
