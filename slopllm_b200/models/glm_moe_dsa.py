"""glm_moe_dsa: MLA latent attention + DSA sparse-attention indexer + sigmoid MoE + MTP head.

One model definition runs on the fp32 reference op set (CPU, gloo ranks) and on the
sm_100a kernel op set (GPU, NCCL + in-kernel NVLink collectives); the op set and the
communicator are injected.  Layer math follows `src/glm51_model.ts:577-942` (layer),
`:979-1003` (stack), `:1009-1065` (MTP layer); tensor-parallel sharding follows `:178-232`.

Collective placement (explicit, two per layer as in the reference):
  o_proj partial  --all-reduce + residual add + RMSNorm-->  MLP input
  MLP partial     --all-reduce + residual add + RMSNorm-->  next layer's attention input
Under context parallelism (`cp`) each rank keeps every `W`-th token's KV row, attends
with all heads over its shard and the partial (o, lse) are merged by log-sum-exp into a
head-sharded output; the indexer's per-rank top-k lists are merged into the global top-k.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ..config import GlmMoeDsaConfig, PAGE_SIZE, env_flag
from ..parallel.dist import Comm, ParallelContext
from ..utils.tracing import traced

EP_ALL_TO_ALL = env_flag("EP_A2A")      # expert parallelism by token dispatch / combine over NCCL instead of masked partial sums
EP_FUSED_MIN_T = 33                     # from this many token rows on `--ep` dispatches / combines in kernels over peer memory
from .weights import LayerWeights, ModelWeights


@dataclass
class LayerCache:
    kv: torch.Tensor                      # u8 [num_slots, kv_row_bytes]
    idx: Optional[torch.Tensor] = None    # u8 [num_slots, index_head_dim + 4] (full-indexer layers)


@dataclass
class KVCacheTensors:
    """Per-layer paged caches.  Slot = page_id * PAGE_SIZE + offset; with CP each rank
    stores the rows of the tokens it owns, so a page id covers PAGE_SIZE * W tokens."""

    layers: List[LayerCache]
    num_pages: int
    page_size: int = PAGE_SIZE

    @classmethod
    def allocate(cls, cfg: GlmMoeDsaConfig, num_pages: int, device, num_layers: Optional[int] = None) -> "KVCacheTensors":
        n = cfg.num_hidden_layers + cfg.num_nextn_predict_layers if num_layers is None else num_layers
        layers = []
        for i in range(n):
            kv = torch.zeros(num_pages * PAGE_SIZE, cfg.kv_row_bytes, dtype=torch.uint8, device=device)
            idx = None
            if cfg.indexer_is_full(i):
                idx = torch.zeros(num_pages * PAGE_SIZE, cfg.index_row_bytes, dtype=torch.uint8, device=device)
            layers.append(LayerCache(kv, idx))
        return cls(layers, num_pages)

    def nbytes(self) -> int:
        return sum(l.kv.numel() + (l.idx.numel() if l.idx is not None else 0) for l in self.layers)


@dataclass
class StepState:
    """Device-side metadata of one forward step (the reference's `ExecutionState`,
    `src/execution-workspace.ts:71-390`)."""

    input_ids: torch.Tensor               # [T]
    positions: torch.Tensor               # [T] int32, global position of each token
    batch_idx: torch.Tensor               # [T] int32, sequence (row of page_table) of each token
    page_table: torch.Tensor              # [B, P] int32 page ids
    logits_idx: Optional[torch.Tensor] = None   # token indices whose logits are wanted (None = all)
    page_size: int = PAGE_SIZE
    cp_world: int = 1
    cp_rank: int = 0
    # carried between layers: slots chosen by the last full-indexer layer
    slots: Optional[torch.Tensor] = None
    lengths: Optional[torch.Tensor] = None
    max_kv_len: int = 0                   # host-side bound on positions + 1 (kernel planning)
    extra: dict = field(default_factory=dict)

    @property
    def num_tokens(self) -> int:
        return self.input_ids.shape[0]


class GlmMoeDsaModel:
    def __init__(self, cfg: GlmMoeDsaConfig, weights: ModelWeights, ctx: Optional[ParallelContext] = None,
                 ops=None, comm: Optional[Comm] = None):
        from ..ops import get_ops
        self.cfg = cfg
        self.w = weights
        self.ctx = ctx or ParallelContext(device=weights.embed.device)
        self.ops = ops or get_ops(cfg, weights.embed.device, self.ctx)
        self.comm = comm or Comm(self.ctx)
        # context parallelism, two forms over the same token-interleaved cache.  Merge: every rank scores and attends over
        # its own shard for all heads, top-k candidates and attention partials are merged across the ranks.  Gather: each
        # layer's rows are all-gathered into a flat buffer and every rank attends like a TP rank over its own heads.
        # On NVLink the gather is cheap (a few tens of MB per layer and chunk) and the 8-head attention kernel is far
        # more efficient than the 64-head one the merge form needs, so prefill-sized steps gather (128K tokens on
        # 4 x B200: 16.8 s against 23.2 s); decode steps, whose per-step gather would move the whole context, merge.
        # SLOPLLM_B200_CP_GATHER_KV=1 / 0 forces one form for every step.
        from ..config import env_str
        self.cp_gather_mode = env_str("CP_GATHER_KV")
        # SLOPLLM_B200_L2_PREFETCH=1: decode steps pull the next layer's attention / router weights into L2 on a side
        # stream while the current layer's experts stream.  Off by default: on B200 it measured 3 % slower at batch 1 and
        # batch 8 (7.82 vs 7.57 ms and 12.67 vs 12.21 ms per 78-layer step of one TP-8 rank), the extra grid costs more
        # than the L2 hits give back
        self.l2_prefetch = env_str("L2_PREFETCH") == "1" and self.w.embed.is_cuda
        self._pf_sets = {}
        self._pf_stream = None

    # -- context parallelism, gather-KV mode ------------------------------------------------
    CP_GATHER_MIN_ROWS = 33        # steps of at least this many rows gather the KV rows (CUDA, no override)

    def _cp_gathers(self, st: StepState) -> bool:
        if self.cp_gather_mode in ("0", "1"):
            return self.cp_gather_mode == "1"
        return st.input_ids.is_cuda and st.input_ids.shape[0] >= self.CP_GATHER_MIN_ROWS

    def _gathered_view(self, lc: LayerCache, st: StepState, with_index: bool = True):
        """Flat replicated copy of the step's sequences' rows of one layer, and a StepState that addresses it.

        Every rank reads its local rows (local index i of sequence b = global position i*W + r) through the page
        table, the ranks all-gather them and interleave so that row b*L + p of the flat buffer is global position
        p.  The returned state has an identity page table and no CP, so the ordinary TP attention path runs on it.
        Reference: `gatherPages` + all-gather + `deinterleave` (`src/parallel_ops.ts:4139-4203`), the reference's
        gather-KV mode (`shouldGatherKv`, `src/glm51_model.ts:380-413`)."""
        W = st.cp_world
        ps = st.page_size
        B = st.page_table.shape[0]
        n_local = -(-max(1, st.max_kv_len) // W)
        n_local = -(-n_local // ps) * ps                                   # whole pages
        dev = lc.kv.device
        i = torch.arange(n_local, device=dev)
        slots = (st.page_table[:, : n_local // ps].long().repeat_interleave(ps, dim=1) * ps + (i % ps).unsqueeze(0)).reshape(-1)

        def flat(cache_t):
            rows = cache_t[slots].view(B, n_local, -1)                      # this rank's rows, local order
            allr = torch.stack(self.comm.all_gather_list(rows.contiguous()), dim=2)     # [B, n_local, W, bytes]
            return allr.reshape(B * n_local * W, -1)                        # position p = i*W + r -> row b*L + p

        L = n_local * W
        table = (torch.arange(B, device=dev).unsqueeze(1) * (L // ps) + torch.arange(L // ps, device=dev).unsqueeze(0)).to(torch.int32)
        st2 = StepState(input_ids=st.input_ids, positions=st.positions, batch_idx=st.batch_idx, page_table=table.contiguous(),
                        logits_idx=st.logits_idx, page_size=ps, cp_world=1, cp_rank=0, slots=st.slots, lengths=st.lengths,
                        max_kv_len=st.max_kv_len, extra=st.extra)
        return LayerCache(flat(lc.kv), flat(lc.idx) if (lc.idx is not None and with_index) else None), st2

    # -- attention -------------------------------------------------------------------------
    @traced("attention")
    def attention(self, layer: int, lw: LayerWeights, x: torch.Tensor, st: StepState, cache: KVCacheTensors):
        ops, comm, ctx = self.ops, self.comm, self.ctx
        lc = cache.layers[layer]
        qkv = ops.linear(x, lw.w_qkv_a, defer_reduce=True)
        cq, idx_w = ops.attn_pre(qkv, lw, st, lc)
        qb = ops.linear(cq, lw.w_q_b, defer_reduce=True)
        q_abs, q_pe, q8, w_eff = ops.q_post(qb, lw, st, idx_w)
        if ctx.cp and ctx.world > 1 and self._cp_gathers(st):
            # the index keys stay sharded when the communicator can return every rank's winners: each rank scores its own
            # shard, the candidates' scores and positions are gathered and re-selected (1 / W of the scoring work per rank)
            sharded_index = lw.has_indexer and hasattr(comm, "cp_merge_topk_all")
            flat_lc, fst = self._gathered_view(lc, st, with_index=not sharded_index)
            if lw.has_indexer:
                if sharded_index:
                    pos, score = ops.indexer_topk(q8, w_eff, lc, st)
                    st.extra.pop("fused_slots", None)
                    pos = comm.cp_merge_topk_all(ops, pos, score, self.cfg.index_topk)
                else:
                    pos, _ = ops.indexer_topk(q8, w_eff, flat_lc, fst)
                fst.slots, fst.lengths = ops.topk_to_slots(pos, fst)
                st.slots, st.lengths = fst.slots, fst.lengths           # flat-buffer slots are valid for the sharing layers too
            elif st.slots is None:
                raise RuntimeError(f"layer {layer} shares indexer slots but no full-indexer layer ran before it")
            return ops.linear(self._attn_values(q_abs, q_pe, flat_lc, st, lw), lw.o_proj, out_f32=True,
                              sink=comm.partial_sink(x.shape[0]))
        if lw.has_indexer:
            pos, score = ops.indexer_topk(q8, w_eff, lc, st)
            if ctx.cp and ctx.world > 1:
                pos = comm.cp_merge_topk(ops, pos, score, self.cfg.index_topk)
            st.slots, st.lengths = ops.topk_to_slots(pos, st, local_only=ctx.cp)
        elif st.slots is None:
            raise RuntimeError(f"layer {layer} shares indexer slots but no full-indexer layer ran before it")
        if ctx.cp and ctx.world > 1:
            q_abs, q_pe = comm.all_gather_many([q_abs, q_pe], dim=1)          # both query parts in one collective
            if hasattr(ops, "sparse_mla_partials"):
                o = comm.cp_merge_partials(ops, *ops.sparse_mla_partials(q_abs, q_pe, lc, st.slots, st.lengths))
            else:
                o, lse = ops.sparse_mla(q_abs, q_pe, lc, st.slots, st.lengths)
                o = comm.cp_merge_heads(ops, o, lse)
            return ops.linear(ops.v_expand(o, lw.w_v), lw.o_proj, out_f32=True, sink=comm.partial_sink(x.shape[0]))
        return ops.linear(self._attn_values(q_abs, q_pe, lc, st, lw), lw.o_proj, out_f32=True, sink=comm.partial_sink(x.shape[0]))

    def _attn_values(self, q_abs, q_pe, lc, st, lw):
        ops = self.ops
        if hasattr(ops, "attn_values"):
            return ops.attn_values(q_abs, q_pe, lc, st.slots, st.lengths, lw.w_v)
        o, _ = ops.sparse_mla(q_abs, q_pe, lc, st.slots, st.lengths)
        return ops.v_expand(o, lw.w_v)

    # -- MLP ----------------------------------------------------------------------------------
    @traced("mlp")
    def mlp(self, lw: LayerWeights, y: torch.Tensor, final: bool = False):
        ops, ctx = self.ops, self.ctx
        if lw.experts is not None and ctx.ep and ctx.world > 1:
            if EP_ALL_TO_ALL:
                return self._moe_ep(lw, y)
            if y.shape[0] >= EP_FUSED_MIN_T and self._ep_exchange_for(lw, y) is not None:
                out = self._moe_ep_fused(lw, y)
                sink = self.comm.partial_sink(y.shape[0], final=final)
                return out if sink is None else sink.push_tensor(out)
            out = self._moe_ep_partial(lw, y)
            sink = self.comm.partial_sink(y.shape[0], final=final)
            return out if sink is None else sink.push_tensor(out)
        sink = self.comm.partial_sink(y.shape[0], final=final)
        if lw.experts is None:
            return ops.dense_mlp(y, lw, sink=sink)
        return ops.moe_tp(y, lw, sink=sink)

    def _moe_ep_partial(self, lw: LayerWeights, y: torch.Tensor):
        """Expert parallelism without a dispatch: the normed hidden rows are replicated on every rank of the replica, so
        each rank routes all of them, runs the routes that land on the experts it owns (full-width experts, the others
        masked out) plus its column slice of the shared expert, and returns that as its partial sum; the all-reduce that
        follows every MLP anyway adds the ranks' contributions up.  No all-to-all, no host synchronisation, fixed shapes:
        the step stays capturable in a CUDA graph and its partial sum can go through the fused NVLink all-reduce.
        (`SLOPLLM_B200_EP_A2A=1` selects the token-split dispatch / combine form below instead.)"""
        ops, ctx = self.ops, self.ctx
        ids, wts = ops.route(y, lw)
        lo = lw.experts.expert_offset
        mine = (ids >= lo) & (ids < lo + lw.experts.num_experts)
        out = ops.moe_local_experts(y, lw.experts, torch.where(mine, ids, torch.full_like(ids, -1)),
                                    torch.where(mine, wts, torch.zeros_like(wts)))
        if lw.shared is not None:
            out = out + ops.shared_expert(y, lw).to(out.dtype)
        return out

    EP_MAX_TOKENS = 8192       # most token rows of one forward that the fused exchange's buffers are sized for

    def _ep_exchange_for(self, lw: LayerWeights, y: torch.Tensor):
        """The peer-memory exchange of this model (made on first use), or None where the fused path does not apply: not on
        CUDA, weights not NVFP4 or of shapes the block-scaled kernels do not take, more rows than the buffers hold."""
        if getattr(self, "_ep_exchange", None) is not None:
            return self._ep_exchange if y.shape[0] <= self.EP_MAX_TOKENS else None
        if getattr(self, "_ep_unavailable", False) or not y.is_cuda or env_flag("EP_NO_FUSED"):
            return None
        from ..ops.gemm import fp4_moe_ok
        if not fp4_moe_ok(lw.experts, self.cfg.hidden_size) or y.shape[0] > self.EP_MAX_TOKENS:
            self._ep_unavailable = not fp4_moe_ok(lw.experts, self.cfg.hidden_size)
            return None
        from ..parallel.ep import make_exchange
        self._ep_exchange = make_exchange(self.ctx, self.cfg, self.EP_MAX_TOKENS)
        return self._ep_exchange

    def _moe_ep_fused(self, lw: LayerWeights, y: torch.Tensor):
        """Expert parallelism with the exchange in kernels: each rank is home to a slice of the rows, stores the 4-bit copy
        of every routed row into its expert's owner over NVLink, the owners run their experts as block-scaled grouped GEMMs
        whose epilogue stores the results back into the home rank, which sums them with the routing weights
        (`parallel/ep.py`).  The result holds the home rows only (plus this rank's slice of the shared expert for all
        rows), so the all-reduce that follows also acts as the all-gather of the rows."""
        ops, ctx = self.ops, self.ctx
        W, r = ctx.world, ctx.rank
        T = y.shape[0]
        per = -(-T // W)
        lo, hi = min(T, r * per), min(T, (r + 1) * per)
        yb = y if y.dtype == torch.bfloat16 else y.to(torch.bfloat16)
        x_loc = yb[lo:hi].contiguous()
        ids, wts = ops.route(x_loc, lw) if hi > lo else (torch.zeros(0, self.cfg.num_experts_per_tok, dtype=torch.int32, device=y.device),
                                                         torch.zeros(0, self.cfg.num_experts_per_tok, device=y.device))
        out = ops.shared_expert(yb, lw).to(torch.float32) if lw.shared is not None else torch.zeros(T, y.shape[1], dtype=torch.float32, device=y.device)
        if not out.is_contiguous():
            out = out.contiguous()
        self._ep_exchange.moe(x_loc, lw.experts, ids, wts, out[lo:hi], accumulate=True)
        return out

    def _moe_ep(self, lw: LayerWeights, y: torch.Tensor):
        """Expert parallelism: tokens are split across ranks, each token's hidden row is
        dispatched to the ranks owning its experts, expert outputs come back weighted and
        are summed at the token's home rank.  The result is written into this rank's
        token slice of the partial sum, so the following all-reduce also acts as the
        token all-gather."""
        ops, comm, ctx = self.ops, self.comm, self.ctx
        W, r = ctx.world, ctx.rank
        T = y.shape[0]
        per = -(-T // W)
        lo, hi = min(T, r * per), min(T, (r + 1) * per)
        x_loc = y[lo:hi]
        ids, wts = ops.route(x_loc, lw)
        E_per = self.cfg.n_routed_experts // W
        owner = torch.div(ids.to(torch.int64), E_per, rounding_mode="floor")      # [t, k]
        send_x, send_ids, send_w, send_tok = [], [], [], []
        for peer in range(W):
            hit = owner == peer
            tok = hit.any(1).nonzero(as_tuple=True)[0]
            send_tok.append(tok)
            send_x.append(x_loc[tok])
            send_ids.append(torch.where(hit[tok], ids[tok], torch.full_like(ids[tok], -1)))
            send_w.append(torch.where(hit[tok], wts[tok], torch.zeros_like(wts[tok])))
        rx = comm.all_to_all(send_x)
        rid = comm.all_to_all(send_ids)
        rw = comm.all_to_all(send_w)
        outs = []
        for peer in range(W):
            if rx[peer].shape[0] == 0:
                outs.append(torch.zeros(0, y.shape[1], dtype=y.dtype, device=y.device))
                continue
            outs.append(ops.moe_local_experts(rx[peer], lw.experts, rid[peer], rw[peer]).to(y.dtype))
        back = comm.all_to_all(outs)
        out = ops.shared_expert(y, lw).to(y.dtype) if lw.shared is not None else torch.zeros_like(y)
        for peer in range(W):
            if back[peer].shape[0]:
                out[lo:hi].index_add_(0, send_tok[peer], back[peer].to(out.dtype))
        return out

    # -- stack -----------------------------------------------------------------------------------
    @traced(lambda self, layer, *a, **k: f"layer{layer}")
    def _layer(self, layer: int, lw: LayerWeights, partial, residual, st, cache, first: bool, last: bool = False):
        ops, comm = self.ops, self.comm
        if first:
            x, residual = ops.add_rmsnorm(partial, residual, lw.input_norm)
        else:
            x, residual = comm.allreduce_add_rmsnorm(ops, partial, residual, lw.input_norm, self.cfg.rms_norm_eps)
        attn = self.attention(layer, lw, x, st, cache)
        y, residual = comm.allreduce_add_rmsnorm(ops, attn, residual, lw.post_attn_norm, self.cfg.rms_norm_eps, want_perm=True)
        if st.extra.get("l2_prefetch") and not last:
            self._prefetch_layer(layer + 1)
        return self.mlp(lw, y, final=last), residual

    # -- L2 prefetch of the next layer (decode) ------------------------------------------------------
    def _prefetch_layer(self, layer: int) -> None:
        """The weights every token of layer `layer` will read (attention projections, absorb / value matrices, router,
        shared expert; not the routed experts, which are not known yet) go to L2 from a side stream while the current
        layer's MLP runs: at decode the main chain is latency-bound and leaves most of the HBM bandwidth idle.
        Reference: `prefetch_l2` ahead of the next layer (`csrc/glm_ops.cu`)."""
        from ..ops.misc import PrefetchSet
        ps = self._pf_sets.get(layer)
        if ps is None:
            lw = self.w.layers[layer]
            ts = [lw.w_qkv_a.weight, lw.w_q_b.weight, lw.w_kn, lw.w_v, lw.o_proj.weight, lw.o_proj.scale]
            if getattr(lw, "router_w", None) is not None:
                ts.append(lw.router_w)
                sh = getattr(lw, "shared", None)
                if sh is not None:
                    ts += [sh.w13, sh.s13, sh.w2, sh.s2]
            ps = self._pf_sets[layer] = PrefetchSet(ts)
        if self._pf_stream is None:
            self._pf_stream = torch.cuda.Stream(device=self.w.embed.device)
        main = torch.cuda.current_stream()
        self._pf_stream.wait_stream(main)
        ps.launch(self._pf_stream)

    def _join_prefetch(self) -> None:
        if self._pf_stream is not None:
            torch.cuda.current_stream().wait_stream(self._pf_stream)

    def forward_hidden(self, st: StepState, cache: KVCacheTensors) -> torch.Tensor:
        """Token ids -> final-normed hidden states [T, H] (replicated on every rank)."""
        ops = self.ops
        partial, residual = ops.embed(st.input_ids, self.w.embed), None
        st.slots = st.lengths = None
        self.comm.begin_forward()
        n = self.cfg.num_hidden_layers
        st.extra["l2_prefetch"] = self.l2_prefetch and st.input_ids.is_cuda and st.input_ids.shape[0] <= 32
        for i in range(n):
            partial, residual = self._layer(i, self.w.layers[i], partial, residual, st, cache, first=(i == 0), last=(i == n - 1))
        if st.extra["l2_prefetch"]:
            self._join_prefetch()              # the side stream rejoins (a captured step must end on one stream)
        hidden, _ = self.comm.allreduce_add_rmsnorm(ops, partial, residual, self.w.final_norm, self.cfg.rms_norm_eps)
        return hidden

    def forward_hidden_phased(self, sts, cache: KVCacheTensors, streams=None):
        """Phased prefill: the chunk is cut into consecutive parts (normally two halves) that walk the layers
        in lock step, part p on `streams[p]`.  Part p+1 starts layer i once part p has finished it (its KV
        rows of that layer are then in the cache), so one part's collectives run under the other part's
        GEMMs.  With `streams=None` the parts simply alternate on the current stream (CPU, tests).
        Returns the parts' hidden states.  Reference: `forwardPhased` generators driven by
        `planPhasedPrefill` (`src/chat_model.ts:204-282`, `src/glm51_model.ts:979-1003`)."""
        import contextlib
        ops, n, P = self.ops, self.cfg.num_hidden_layers, len(sts)
        use_streams = streams is not None and sts[0].input_ids.is_cuda
        ctx = (lambda p: torch.cuda.stream(streams[p])) if use_streams else (lambda p: contextlib.nullcontext())
        if use_streams:
            start = torch.cuda.Event()
            start.record()
            for s in streams:
                s.wait_event(start)
        partial, residual = [None] * P, [None] * P
        for p, st in enumerate(sts):
            with ctx(p):
                partial[p] = ops.embed(st.input_ids, self.w.embed)
                st.slots = st.lengths = None
        self.comm.begin_forward()
        done = [None] * P
        for i in range(n):
            for p, st in enumerate(sts):
                with ctx(p):
                    if use_streams and p > 0:
                        streams[p].wait_event(done[p - 1])
                    partial[p], residual[p] = self._layer(i, self.w.layers[i], partial[p], residual[p], st, cache,
                                                          first=(i == 0), last=(i == n - 1))
                    if use_streams:
                        done[p] = torch.cuda.Event()
                        done[p].record(streams[p])
        hidden = []
        for p in range(P):
            with ctx(p):
                h, _ = self.comm.allreduce_add_rmsnorm(ops, partial[p], residual[p], self.w.final_norm, self.cfg.rms_norm_eps)
                hidden.append(h)
        if use_streams:
            cur = torch.cuda.current_stream()
            for s in streams:
                cur.wait_stream(s)
        return hidden

    def forward_mtp(self, st: StepState, cache: KVCacheTensors, prev_hidden: torch.Tensor, depth: int = 0) -> torch.Tensor:
        """MTP layer: combines the embedding of the *next* token (st.input_ids) with the
        previous hidden state, runs one decoder layer, returns the head-normed hidden.

        When the MTP layer shares indexer slots, `st.slots` must still hold the slots of
        the main model's last full-indexer layer for the same tokens.
        """
        cfg, ops = self.cfg, self.ops
        li = cfg.num_hidden_layers + min(depth, cfg.num_nextn_predict_layers - 1)
        lw = self.w.layers[li]
        e = ops.rmsnorm(ops.embed(st.input_ids, self.w.embed), lw.enorm)
        g = ops.rmsnorm(prev_hidden, lw.hnorm)
        z = ops.linear(torch.cat([e, g], dim=-1), lw.eh_proj)
        self.comm.begin_forward()
        partial, residual = self._layer(li, lw, z, None, st, cache, first=True, last=True)
        hidden, _ = self.comm.allreduce_add_rmsnorm(ops, partial, residual, lw.shared_head_norm, cfg.rms_norm_eps)
        return hidden

    def compute_logits(self, hidden: torch.Tensor, logits_idx: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Full-vocabulary logits (column-sharded lm_head, then all-gather)."""
        if logits_idx is not None:
            hidden = hidden[logits_idx.to(torch.int64)]
        return self.comm.all_gather(self.ops.logits(hidden, self.w.lm_head), dim=-1)

    def forward(self, st: StepState, cache: KVCacheTensors) -> torch.Tensor:
        return self.compute_logits(self.forward_hidden(st, cache), st.logits_idx)


def make_step(input_ids, positions, batch_idx, page_table, ctx: Optional[ParallelContext] = None,
              logits_idx=None) -> StepState:
    """Build a StepState from host lists / tensors on the model's device."""
    ctx = ctx or ParallelContext()
    dev = ctx.device
    t = lambda v, dt: torch.as_tensor(v, dtype=dt, device=dev)
    pos = t(positions, torch.int32)
    return StepState(
        input_ids=t(input_ids, torch.int64), positions=pos, batch_idx=t(batch_idx, torch.int32),
        page_table=t(page_table, torch.int32), logits_idx=None if logits_idx is None else t(logits_idx, torch.int64),
        cp_world=ctx.cp_world, cp_rank=ctx.cp_rank,
        max_kv_len=int(max(positions)) + 1 if len(positions) else 0,
    )
