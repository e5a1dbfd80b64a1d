"""sm_100a op set: the staged model ops implemented with the in-tree CUDA kernels.

Activations are bf16, the residual stream and partial sums are fp32, caches are packed
bytes.  Every method launches hand-written kernels from `libslopllm_kernels.so` on the
current stream (so the whole step can be captured in a CUDA graph); nothing here falls
back to PyTorch math on the hot path.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import native as N
from . import reference as R

DECODE_MAX_T = 32          # token rows handled by the weight-streaming (GEMV) kernels
TENSOR_MIN_T = 2           # from this many rows on the streaming kernels use the tensor cores


class SplitKSlabs:
    """fp32 partial sums [splits, T, N] of a split-K product; their sum rounded to bf16 is the value."""

    def __init__(self, slabs: torch.Tensor):
        self.slabs = slabs

    @property
    def shape(self):
        return self.slabs.shape[1:]

    @property
    def device(self):
        return self.slabs.device

    def reduce(self) -> torch.Tensor:
        return self.slabs.sum(0).to(torch.bfloat16)


def _act_source(a):
    """(row-0 view, n_slabs, slab_stride) of an activation in either form."""
    if isinstance(a, SplitKSlabs):
        return a.slabs[0], a.slabs.shape[0], a.slabs.stride(0)
    return a, 0, 0


class CudaOps:
    name = "cuda"
    act_dtype = torch.bfloat16

    def __init__(self, cfg, ctx=None):
        self.cfg = cfg
        self.ctx = ctx
        N.kernels()            # fail loudly when the native library is missing
        self._counters = {}
        from ..config import env_str
        # one-launch persistent decode MoE (csrc/moe_persist.cu): opt-in.  Its NVFP4 -> f16 expansion is bound by the
        # conversion rate of the CUDA cores just like the five-launch path, which it does not yet beat below 32 rows
        self._persist_moe = env_str("MOE_PERSIST") == "1"
        self._fused_attn_out = env_str("FUSED_ATTN_OUT") != "0"     # merge of the key splits inside the value expansion
        self._fp4_decode_force = env_str("MOE_FP4_DECODE")          # "0" / "1": never / always the FP4 GEMMs for decode-sized MoE
        self._persist_gsub = 0         # gate/up sub-tiles per tile of the persistent MoE kernel (0: the kernel's default)
        self._persist_trace = None     # u64 [SMs, 96, 4] tile timeline, filled when set (profiling)

    # -- helpers ----------------------------------------------------------------------------
    @staticmethod
    def _bf16(x):
        return x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)

    # -- elementwise / linear ---------------------------------------------------------------
    def embed(self, ids, table):
        T, H = ids.shape[0], table.shape[1]
        out = torch.empty(T, H, dtype=torch.bfloat16, device=table.device)
        ids = ids.to(torch.int64).contiguous()
        N.call("sl_embed", out.data_ptr(), ids.data_ptr(), table.data_ptr(), T, H, table.shape[0], N.stream())
        return out

    def add_rmsnorm(self, x, residual, w, eps=None, want_perm: bool = False):
        eps = self.cfg.rms_norm_eps if eps is None else eps
        x = x.contiguous()
        if x.dtype not in (torch.bfloat16, torch.float32):
            x = x.to(torch.float32)
        T, H = x.shape
        out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
        res = torch.empty(T, H, dtype=torch.float32, device=x.device)
        xp = None
        if want_perm and T <= DECODE_MAX_T and H % 128 == 0:
            # the consumer is an NVFP4 tensor-core kernel: write its permuted f16 operand in the same pass
            xp = torch.empty(((T + 7) // 8) * 8 * H, dtype=torch.float16, device=x.device)
            out._sl_perm = xp
        N.call("sl_add_rmsnorm", out.data_ptr(), res.data_ptr(), x.data_ptr(), N.ptr(residual), w.data_ptr(), T, H,
               float(eps), int(x.dtype == torch.float32), N.ptr(xp), N.stream())
        return out, res

    @staticmethod
    def _perm_of(x, T: int, K: int):
        """The permuted f16 copy that x's producer left with it, if it has the shape this consumer needs."""
        p = getattr(x, "_sl_perm", None)
        return p if p is not None and p.numel() == ((T + 7) // 8) * 8 * K else None

    def rmsnorm(self, x, w, eps=None):
        eps = self.cfg.rms_norm_eps if eps is None else eps
        x = x.contiguous()
        T, H = x.shape
        out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
        N.call("sl_add_rmsnorm", out.data_ptr(), 0, x.data_ptr(), 0, w.data_ptr(), T, H, float(eps),
               int(x.dtype == torch.float32), 0, N.stream())
        return out

    def linear(self, x, w, out_f32: bool = False, sink=None, defer_reduce: bool = False):
        """y = x @ W^T.  With `sink` (a receive buffer on every rank) the fp32 result rows are
        stored straight into the peers' memory by the producing kernel and the sink is returned.
        With `defer_reduce` a split-K product may come back as `SplitKSlabs` (fp32 partial sums the
        consumer adds up while it loads them); only `attn_pre` and `q_post` accept that form."""
        x = self._bf16(x)
        if x.stride(-1) != 1:
            x = x.contiguous()
        T, K = x.shape
        Nn = w.out_features
        if getattr(w, "is_fp8", False):
            return self._linear_fp8(x, w, out_f32, sink)
        if sink is not None and hasattr(sink, "rs"):
            # prefill-sized partial sum: the GEMM's epilogue sends each tile row to the rank that owns it
            from . import tcgen05
            from .gemm import _weight_bf16, gemm_large
            wb = _weight_bf16(w)
            if (T == sink.rows and Nn == sink.rs.row_len and K % 8 == 0 and x.stride(0) % 8 == 0 and wb.stride(-1) == 1
                    and wb.stride(0) % 8 == 0):
                N.call("sl_gemm_bf16_tcgen05_rs", x.data_ptr(), wb.data_ptr(), T, Nn, K, x.stride(0), wb.stride(0),
                       tcgen05.error_flag(x.device).data_ptr(), 256 if Nn >= 512 else 128, C.byref(sink.rs), N.stream())
                return sink
            return sink.push_tensor(gemm_large(x, w, True))
        if sink is not None:
            sink.pushed_rows = T
            if w.is_nvfp4 and K % 128 == 0 and x.stride(0) % 8 == 0:
                xp = self._perm_of(x, T, K)
                ready = xp is not None
                if not ready:
                    xp = torch.empty(((T + 7) // 8) * 8 * K, dtype=torch.float16, device=x.device)
                N.call("sl_linear_nvfp4_mma_push", 0 if ready else x.data_ptr(), xp.data_ptr(), w.weight.data_ptr(),
                       w.scale.data_ptr(), w.scale2.data_ptr(), T, Nn, K, K if ready else x.stride(0), C.byref(sink.push), N.stream())
                return sink
            if not w.is_nvfp4 and x.stride(0) % 8 == 0 and K % 8 == 0:
                from . import tcgen05
                N.call("sl_linear_smallT_bf16_tcgen05_push", x.data_ptr(), w.weight.data_ptr(), T, Nn, K, x.stride(0),
                       w.weight.stride(0), tcgen05.error_flag(x.device).data_ptr(), C.byref(sink.push), N.stream())
                return sink
            return sink.push_tensor(self.linear(x, w, out_f32=True))
        if T > DECODE_MAX_T:
            from .gemm import gemm_large
            return gemm_large(x, w, out_f32)
        y = torch.empty(T, Nn, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
        if T >= TENSOR_MIN_T:
            # tensor-core weight streaming: tcgen05 swap-AB (bf16) / mma.sync with in-register FP4 expansion
            if w.is_nvfp4 and K % 128 == 0 and x.stride(0) % 8 == 0:
                xp = self._perm_of(x, T, K)
                ready = xp is not None
                if not ready:
                    xp = torch.empty(((T + 7) // 8) * 8 * K, dtype=torch.float16, device=x.device)
                N.call("sl_linear_nvfp4_mma", y.data_ptr(), 0 if ready else x.data_ptr(), xp.data_ptr(), w.weight.data_ptr(),
                       w.scale.data_ptr(), w.scale2.data_ptr(), T, Nn, K, K if ready else x.stride(0), int(out_f32), N.stream())
                return y
            if not w.is_nvfp4 and x.stride(0) % 8 == 0 and K % 8 == 0 and Nn > 1024:
                from . import tcgen05
                splits = N.kernels().sl_smallT_splits(T, Nn, K)
                part = torch.empty(splits, T, Nn, dtype=torch.float32, device=x.device) if splits > 1 else None
                deferred = defer_reduce and splits > 1
                N.call("sl_linear_smallT_bf16_tcgen05", x.data_ptr(), w.weight.data_ptr(), 0 if deferred else y.data_ptr(),
                       T, Nn, K, x.stride(0), w.weight.stride(0), y.stride(0), int(out_f32),
                       tcgen05.error_flag(x.device).data_ptr(), N.ptr(part), splits, N.stream())
                return SplitKSlabs(part) if deferred else y
        if w.is_nvfp4:
            N.call("sl_gemv_nvfp4", y.data_ptr(), x.data_ptr(), w.weight.data_ptr(), w.scale.data_ptr(),
                   w.scale2.data_ptr(), T, Nn, K, x.stride(0), int(out_f32), N.stream())
        else:
            N.call("sl_gemv_bf16", y.data_ptr(), x.data_ptr(), w.weight.data_ptr(), T, Nn, K, x.stride(0), int(out_f32),
                   N.stream())
        return y

    FP8_GEMV_MAX_T = 8         # token rows served by the FP8 weight-streaming kernel in one pass over the weights

    def _linear_fp8(self, x, w, out_f32: bool, sink=None):
        """FP8 block-scaled weight (e4m3 + one scale per 128 x 128 block).  Up to `FP8_GEMV_MAX_T` rows stream the FP8
        bytes directly; more rows expand the matrix to bf16 once and take the tensor-core GEMM paths."""
        from ..models.weights import LinearWeight
        T, K = x.shape
        Nn = w.out_features
        w8, sc = w.weight, w.fp8_scale
        ok = K % 16 == 0 and w8.is_contiguous() and sc.dtype == torch.float32 and sc.is_contiguous()
        if sink is None and ok and T <= self.FP8_GEMV_MAX_T and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0:
            y = torch.empty(T, Nn, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
            N.call("sl_linear_fp8_block", x.data_ptr(), w8.data_ptr(), sc.data_ptr(), y.data_ptr(), T, Nn, K, x.stride(0), Nn,
                   sc.shape[1], int(out_f32), N.stream())
            return y
        if ok:
            wb = torch.empty(Nn, K, dtype=torch.bfloat16, device=x.device)
            N.call("sl_fp8_block_dequant_bf16", wb.data_ptr(), w8.data_ptr(), sc.data_ptr(), Nn, K, sc.shape[1], N.stream())
        else:
            wb = w.dequant(torch.bfloat16)
        return self.linear(x, LinearWeight(wb), out_f32=out_f32, sink=sink)

    def merge_attention_partials(self, o, lse):
        return R.merge_attention_partials(o, lse)

    # -- attention stages ---------------------------------------------------------------------
    def attn_pre(self, qkv, lw, st, layer_cache):
        c = self.cfg
        T = qkv.shape[0]
        dev = qkv.device
        cq = torch.empty(T, c.q_lora_rank, dtype=torch.bfloat16, device=dev)
        idx_w = torch.empty(T, c.index_n_heads, dtype=torch.float32, device=dev) if lw.has_indexer else None
        qkv, n_slabs, slab_stride = _act_source(qkv)
        p = N.AttnPreParams(
            n_slabs=n_slabs, slab_stride=slab_stride, qkv=qkv.data_ptr(), ld=qkv.stride(0), q_lora=c.q_lora_rank, kv_lora=c.kv_lora_rank, rope_dim=c.qk_rope_head_dim,
            idx_dim=c.index_head_dim if lw.has_indexer else 0, idx_heads=c.index_n_heads,
            q_norm_w=lw.q_a_norm.data_ptr(), kv_norm_w=lw.kv_a_norm.data_ptr(), idx_ln_w=N.ptr(lw.idx_k_norm_w),
            idx_ln_b=N.ptr(lw.idx_k_norm_b), eps=c.rms_norm_eps, theta=c.rope_theta,
            rope_interleave=int(c.rope_interleave), idx_rope_interleave=int(c.indexer_rope_interleave),
            positions=st.positions.data_ptr(), batch_idx=st.batch_idx.data_ptr(), page_table=st.page_table.data_ptr(),
            pt_stride=st.page_table.stride(0), page_size=st.page_size, cp_world=st.cp_world, cp_rank=st.cp_rank,
            kv_group=c.kv_quant_group, kv_cache=layer_cache.kv.data_ptr(), idx_cache=N.ptr(layer_cache.idx),
            cq_out=cq.data_ptr(), idx_w_out=N.ptr(idx_w), num_slots=layer_cache.kv.shape[0], guard=self._guard(dev))
        N.call("sl_attn_pre", C.byref(p), T, N.stream())
        return cq, idx_w

    def q_post(self, qb, lw, st, idx_w):
        c = self.cfg
        T = qb.shape[0]
        dev = qb.device
        hl = lw.w_kn.shape[0]
        q_pe = torch.empty(T, hl, c.qk_rope_head_dim, dtype=torch.bfloat16, device=dev)
        q8 = w_eff = None
        if lw.has_indexer:
            q8 = torch.empty(T, c.index_n_heads, c.index_head_dim, dtype=torch.uint8, device=dev)
            w_eff = torch.empty(T, c.index_n_heads, dtype=torch.float32, device=dev)
        qb, n_slabs, slab_stride = _act_source(qb)
        p = N.QPostParams(
            n_slabs=n_slabs, slab_stride=slab_stride, qb=qb.data_ptr(), ld=qb.stride(0), heads=hl, d_nope=c.qk_nope_head_dim, rope_dim=c.qk_rope_head_dim,
            idx_heads=c.index_n_heads if lw.has_indexer else 0, idx_dim=c.index_head_dim, theta=c.rope_theta,
            rope_interleave=int(c.rope_interleave), idx_rope_interleave=int(c.indexer_rope_interleave),
            positions=st.positions.data_ptr(), idx_w=N.ptr(idx_w), q_pe_out=q_pe.data_ptr(), q8_out=N.ptr(q8),
            w_eff_out=N.ptr(w_eff))
        if T > DECODE_MAX_T and n_slabs == 0:
            # prefill: the absorb product is a plain batched GEMM (one per head): library bmm, as in the reference
            # (`glm_bmm`, `csrc/glm_ops.cu`); the rotary / quantisation part keeps its own kernel
            N.call("sl_q_post", C.byref(p), T, N.stream())
            q_abs = self._head_batched_gemm(qb, c.qk_head_dim, c.qk_nope_head_dim, lw, "w_kn")
            if q_abs is None:         # shapes the tile walk does not take: library batched product
                q_nope = qb[:, :hl * c.qk_head_dim].view(T, hl, c.qk_head_dim)[..., :c.qk_nope_head_dim]
                q_abs = torch.bmm(q_nope.transpose(0, 1), lw.w_kn).transpose(0, 1).contiguous()
            return q_abs.view(T, hl, c.kv_lora_rank), q_pe, q8, w_eff
        q_abs = torch.empty(T, hl, c.kv_lora_rank, dtype=torch.bfloat16, device=dev)
        N.call("sl_q_post_absorb", C.byref(p), q_abs.data_ptr(), lw.w_kn.data_ptr(), T, c.kv_lora_rank, N.stream())
        return q_abs, q_pe, q8, w_eff

    IDX_SCORE_BUDGET = 2 << 30     # bytes of the transient fp32 score matrix [rows, keys]; more query rows go in blocks

    def indexer_topk(self, q8, w_eff, layer_cache, st):
        """Scores of every query token against its sequence's indexer keys, then the top-k positions.  The score matrix is
        sized by the longest sequence of the step, not by the cache capacity, and a prefill chunk against a very long
        context is scored in blocks of query rows so that the matrix stays within `IDX_SCORE_BUDGET` (reference: the
        sizing rules checked by `tests/test_indexer_sizing.ts`)."""
        c = self.cfg
        T = q8.shape[0]
        dev = q8.device
        W, r = st.cp_world, st.cp_rank
        max_local = max(0, -(-st.max_kv_len // W))
        pos = torch.empty(T, c.index_topk, dtype=torch.int32, device=dev)
        score = torch.empty(T, c.index_topk, dtype=torch.float32, device=dev)
        ld = max(8, (max_local + 7) // 8 * 8)
        rows_per = self.score_rows_per_block(T, ld)
        scores = st.extra.get("idx_scores")
        if scores is None or scores.shape[0] < rows_per or scores.shape[1] < ld:
            scores = torch.empty(rows_per, ld, dtype=torch.float32, device=dev)
            st.extra["idx_scores"] = scores
        slots = lengths = None
        if W == 1:
            # without context parallelism the selected positions are final: look the slots up in the same kernel
            slots = torch.empty(T, c.index_topk, dtype=torch.int32, device=dev)
            lengths = torch.empty(T, dtype=torch.int32, device=dev)
            st.extra["fused_slots"] = (pos, slots, lengths)
        for t0 in range(0, T, rows_per):
            t1 = min(T, t0 + rows_per)
            n = t1 - t0
            positions, batch_idx = st.positions[t0:t1], st.batch_idx[t0:t1]
            if st.max_kv_len > c.index_topk:
                sp = N.IndexerScoreParams(
                    q8=q8[t0:t1].data_ptr(), w_eff=w_eff[t0:t1].data_ptr(), idx_cache=layer_cache.idx.data_ptr(),
                    page_table=st.page_table.data_ptr(), pt_stride=st.page_table.stride(0), batch_idx=batch_idx.data_ptr(),
                    positions=positions.data_ptr(), Hi=c.index_n_heads, D=c.index_head_dim, page_size=st.page_size,
                    cp_world=W, cp_rank=r, top_k=c.index_topk, scores=scores.data_ptr(), ld_scores=scores.stride(0),
                    num_slots=layer_cache.idx.shape[0], guard=self._guard(dev),
                    one_sequence=int(bool(st.extra.get("one_sequence", False))), err=self._guard(dev) - 16)
                N.call("sl_indexer_scores", C.byref(sp), n, max_local, N.stream())
            tp = N.TopkSelectParams(scores=scores.data_ptr(), ld_scores=scores.stride(0), positions=positions.data_ptr(),
                                    top_k=c.index_topk, cp_world=W, cp_rank=r, out_pos=pos[t0:t1].data_ptr(),
                                    out_score=score[t0:t1].data_ptr())
            if W == 1:
                tp.slots, tp.lengths = slots[t0:t1].data_ptr(), lengths[t0:t1].data_ptr()
                tp.page_table, tp.batch_idx = st.page_table.data_ptr(), batch_idx.data_ptr()
                tp.pt_stride, tp.page_size = st.page_table.stride(0), st.page_size
            N.call("sl_topk_select", C.byref(tp), n, N.stream())
        return pos, score

    @classmethod
    def score_rows_per_block(cls, T: int, ld: int) -> int:
        """Query rows scored per launch: all of them while [T, ld] fp32 fits the budget, else a multiple of 8 rows."""
        if T * ld * 4 <= cls.IDX_SCORE_BUDGET:
            return max(1, T)
        return max(8, cls.IDX_SCORE_BUDGET // (ld * 4) // 8 * 8)

    def topk_select_plain(self, scores: torch.Tensor, k: int) -> torch.Tensor:
        """Indices of the k largest entries of each row (ascending index order, ties to the lower index, -1 padded
        when a row has fewer than k entries).  scores fp32 [T, n], row stride a multiple of 4 bytes."""
        T, n = scores.shape
        out = torch.empty(T, k, dtype=torch.int32, device=scores.device)
        sc = torch.empty(T, k, dtype=torch.float32, device=scores.device)
        tp = N.TopkSelectParams(scores=scores.data_ptr(), ld_scores=scores.stride(0), positions=0, top_k=k, cp_world=1, cp_rank=0,
                                out_pos=out.data_ptr(), out_score=sc.data_ptr(), n_fixed=n)
        N.call("sl_topk_select", C.byref(tp), T, N.stream())
        return out

    def topk_to_slots(self, topk_pos, st, local_only: bool = False):
        fused = st.extra.pop("fused_slots", None)
        if fused is not None and fused[0] is topk_pos:
            return fused[1], fused[2]
        T, k = topk_pos.shape
        dev = topk_pos.device
        slots = torch.empty(T, k, dtype=torch.int32, device=dev)
        lengths = torch.empty(T, dtype=torch.int32, device=dev)
        topk_pos = topk_pos.contiguous()
        N.call("sl_topk_to_slots", slots.data_ptr(), lengths.data_ptr(), topk_pos.data_ptr(), st.page_table.data_ptr(),
               st.batch_idx.data_ptr(), T, k, st.page_table.stride(0), st.page_size, st.cp_world, st.cp_rank,
               int(local_only), self._guard(dev), N.stream())
        return slots, lengths

    def _mla_splits(self, T: int, h: int) -> int:
        """Split the selected keys so that the grid fills the 148 SMs a few times over
        (the reference's `sparseMlaChunksPerBlock`, `src/sparse-mla-planner.ts:1-21`)."""
        from ..runtime.planner import sparse_mla_splits
        c = self.cfg
        splits = sparse_mla_splits(T, h, c.index_topk)
        if splits > 1 and N.kernels().sl_sparse_mla_tcgen05_decode_ok(c.kv_lora_rank, c.kv_quant_group, c.qk_rope_head_dim, h,
                                                                      c.index_topk):
            splits = max(2, min(splits, (c.index_topk + 127) // 128))      # the tcgen05 kernel's unit of work is a 128-key tile
        return splits

    def sparse_mla_partials(self, q_abs, q_pe, layer_cache, slots, lengths):
        c = self.cfg
        T, h, Rr = q_abs.shape
        dev = q_abs.device
        splits = self._mla_splits(T, h)
        o_part = torch.empty(T, h, splits, Rr, dtype=torch.float32, device=dev)
        lse_part = torch.empty(T, h, splits, dtype=torch.float32, device=dev)
        p = N.SparseMlaParams(q_abs=q_abs.data_ptr(), q_pe=q_pe.data_ptr(), kv_cache=layer_cache.kv.data_ptr(),
                              slots=slots.data_ptr(), lengths=lengths.data_ptr(), h=h, R=Rr, Dr=c.qk_rope_head_dim,
                              group=c.kv_quant_group, topk=slots.shape[1], splits=splits, sm_scale=c.softmax_scale,
                              o_part=o_part.data_ptr(), lse_part=lse_part.data_ptr(), num_slots=layer_cache.kv.shape[0],
                              guard=self._guard(dev), err=self._guard(dev) - 16)
        c_ok = Rr % 64 == 0 and Rr <= 512 and (Rr + c.qk_rope_head_dim) % 16 == 0
        N.call("sl_sparse_mla_split_mma" if c_ok else "sl_sparse_mla_split", C.byref(p), T, N.stream())
        return o_part, lse_part

    def combine_f32(self, o_parts, lse_parts):
        return self.combine(o_parts, lse_parts, out_f32=True)

    def combine(self, o_parts, lse_parts, head_begin=0, head_count=None, want_lse=True, rows=None, out_f32=False, parity=None):
        """o_parts: list of [T, h, S, R] fp32 buffers (one per rank under CP); `rows` limits the
        token rows processed when the buffers are staging areas with spare capacity."""
        T, h, S, Rr = o_parts[0].shape
        T = T if rows is None else rows
        head_count = h if head_count is None else head_count
        dev = o_parts[0].device
        o = torch.empty(T, head_count, Rr, dtype=torch.float32 if out_f32 else torch.bfloat16, device=dev)
        lse = torch.empty(T, head_count, dtype=torch.float32, device=dev) if want_lse else None
        p = N.CombineParams(n_buf=len(o_parts), parts_per_buf=S, h=h, R=Rr, head_begin=head_begin, head_count=head_count,
                            o_out=o.data_ptr(), lse_out=N.ptr(lse), out_f32=int(out_f32))
        if parity is not None:          # (epoch word address, o stride, lse stride): double-buffered staging, see csrc/sparse_mla.cu
            p.parity_epoch, p.parity_o_stride, p.parity_lse_stride = parity
        for i, (a, b) in enumerate(zip(o_parts, lse_parts)):
            p.o_ptrs[i] = a.data_ptr()
            p.lse_ptrs[i] = b.data_ptr()
        N.call("sl_mla_combine", C.byref(p), T, N.stream())
        return o, lse

    def sparse_mla(self, q_abs, q_pe, layer_cache, slots, lengths):
        c = self.cfg
        T, h, Rr = q_abs.shape
        if (self._mla_splits(T, h) == 1 and Rr % 64 == 0 and (Rr + c.qk_rope_head_dim) % 16 == 0
                and N.kernels().sl_sparse_mla_direct_ok(Rr, c.kv_quant_group, c.qk_rope_head_dim)):
            # enough query rows to fill the GPU without key splits: the attention kernel writes the result itself
            dev = q_abs.device
            o = torch.empty(T, h, Rr, dtype=torch.bfloat16, device=dev)
            lse = torch.empty(T, h, dtype=torch.float32, device=dev)
            p = N.SparseMlaParams(q_abs=q_abs.data_ptr(), q_pe=q_pe.data_ptr(), kv_cache=layer_cache.kv.data_ptr(),
                                  slots=slots.data_ptr(), lengths=lengths.data_ptr(), h=h, R=Rr, Dr=c.qk_rope_head_dim,
                                  group=c.kv_quant_group, topk=slots.shape[1], splits=1, sm_scale=c.softmax_scale,
                                  o_part=0, lse_part=0, num_slots=layer_cache.kv.shape[0], guard=self._guard(dev),
                                  o_final=o.data_ptr(), lse_final=lse.data_ptr(), err=self._guard(dev) - 16)
            N.call("sl_sparse_mla_split_mma", C.byref(p), T, N.stream())
            return o, lse
        o_part, lse_part = self.sparse_mla_partials(q_abs, q_pe, layer_cache, slots, lengths)
        return self.combine([o_part], [lse_part])

    def attn_values(self, q_abs, q_pe, layer_cache, slots, lengths, w_v):
        """Sparse attention followed by the value expansion, [T, h * Dv].  At decode the merge of the key splits is the
        staging step of the expansion (one launch instead of merge + product + operand staging for the output
        projection, whose fragment-ordered copy rides along with the result)."""
        T, h, Rr = q_abs.shape
        splits = self._mla_splits(T, h)
        Dv = w_v.shape[2]
        if not self._fused_attn_out or T > DECODE_MAX_T or splits < 2 or splits > 64 or Rr % 4 != 0 or Dv % 8 != 0:
            o, _ = self.sparse_mla(q_abs, q_pe, layer_cache, slots, lengths)
            return self.v_expand(o, w_v)
        o_part, lse_part = self.sparse_mla_partials(q_abs, q_pe, layer_cache, slots, lengths)
        dev = q_abs.device
        out = torch.empty(T, h * Dv, dtype=torch.bfloat16, device=dev)
        tpad = (T + 7) // 8 * 8
        perm = None
        if T >= TENSOR_MIN_T and (h * Dv) % 128 == 0:
            perm = torch.empty(tpad * h * Dv, dtype=torch.float16, device=dev)
        p = N.CombineExpandParams(o_part=o_part.data_ptr(), lse_part=lse_part.data_ptr(), w_v=w_v.data_ptr(), y=out.data_ptr(),
                                  xp=N.ptr(perm), T=T, tpad=tpad, Hh=h, K=Rr, N=Dv, np=splits)
        N.call("sl_combine_vexpand", C.byref(p), N.stream())
        if perm is not None:
            out._sl_perm = perm
        return out

    def _head_batched_gemm(self, a, a_stride: int, K: int, owner, w):
        """out[t, h * n + j] = sum_k a[t, h * a_stride + k] * W[h, k, j] on the persistent tcgen05 GEMM (`W` [heads, K, n];
        its output-major copy [heads * n, K] is made once and kept on the tensor's owner).  None when the shape is not one
        the tile walk takes.  Replaces the library bmm of the absorb and value-expansion steps of a prefill chunk
        (the reference calls cuBLAS strided-batched there, `csrc/glm_ops.cu` `glm_bmm`)."""
        from . import tcgen05
        if isinstance(w, str):
            name, w = w, getattr(owner, w)
            wt = getattr(owner, "_" + name + "_t", None)
        else:
            name, wt = None, getattr(w, "_sl_out_major", None)
        heads, Kw, n = w.shape
        if (Kw != K or K % 64 != 0 or n % 64 != 0 or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.stride(-1) != 1
                or a.stride(0) % 8 != 0 or a_stride % 8 != 0):
            return None
        if wt is None:
            wt = w.transpose(1, 2).contiguous().view(heads * n, K)
            if name is not None:
                setattr(owner, "_" + name + "_t", wt)
            else:
                w._sl_out_major = wt
        T = a.shape[0]
        out = torch.empty(T, heads * n, dtype=torch.bfloat16, device=a.device)
        N.call("sl_gemm_bf16_tcgen05_batched", a.data_ptr(), wt.data_ptr(), out.data_ptr(), T, heads, n, K, a.stride(0), a_stride,
               K, heads * n, 0, tcgen05.error_flag(a.device).data_ptr(), N.stream())
        return out

    def v_expand(self, o, w_v):
        T, hl, Rr = o.shape
        Dv = w_v.shape[2]
        o = self._bf16(o).contiguous()
        if T > DECODE_MAX_T:
            # prefill: one tcgen05 GEMM walks the (token tile, head) grid; the head's matrix is stored output-major once
            out = self._head_batched_gemm(o.view(T, hl * Rr), Rr, Rr, None, w_v)
            if out is not None:
                return out
            return torch.bmm(o.transpose(0, 1), w_v).transpose(0, 1).reshape(T, hl * Dv)
        out = torch.empty(T, hl * Dv, dtype=torch.bfloat16, device=o.device)
        N.call("sl_bmv", out.data_ptr(), o.data_ptr(), w_v.data_ptr(), T, hl, Rr, Dv, hl * Rr, Rr, 0, 0, N.stream())
        return out

    # -- MLP --------------------------------------------------------------------------------------
    def dense_mlp(self, x, lw, sink=None):
        gu = self.linear(x, lw.mlp_w13)
        if gu.stride(0) != gu.shape[1]:
            gu = gu.contiguous()
        T, I2 = gu.shape
        act = torch.empty(T, I2 // 2, dtype=torch.bfloat16, device=x.device)
        N.call("sl_silu_mul", act.data_ptr(), gu.data_ptr(), T, I2 // 2, N.stream())
        return self.linear(act, lw.mlp_w2, out_f32=True, sink=sink)

    def route(self, x, lw):
        c = self.cfg
        T = x.shape[0]
        E = lw.router_w.shape[0]
        logits = self._router_logits(x, lw)
        ids = torch.empty(T, c.num_experts_per_tok, dtype=torch.int32, device=x.device)
        wts = torch.empty(T, c.num_experts_per_tok, dtype=torch.float32, device=x.device)
        N.call("sl_route_topk", ids.data_ptr(), wts.data_ptr(), logits.data_ptr(), N.ptr(lw.router_bias), T, E,
               c.num_experts_per_tok, c.n_group, c.topk_group, int(c.norm_topk_prob), float(c.routed_scaling_factor),
               N.stream())
        return ids, wts

    def _router_logits(self, x, lw):
        from ..models.weights import LinearWeight
        return self.linear(x, LinearWeight(lw.router_w), out_f32=True)

    def _moe_small(self, x, experts, shared, ids, wts, sink=None):
        """Weight-streaming MoE for a few token rows: gate/up + SiLU·mul per route, then
        down-projection fused with the routing-weighted sum (and the shared expert)."""
        x = self._bf16(x)
        T, H = x.shape
        k = ids.shape[1]
        I = experts.inter
        routes = T * k + (T if shared is not None else 0)
        if H % 128 == 0 and I % 128 == 0 and x.stride(0) % 8 == 0 and T * k <= 480:
            return self._moe_grouped(x, experts, shared, ids, wts, sink)
        act = torch.empty(routes, I, dtype=torch.bfloat16, device=x.device)
        gp = N.MoeGateUpParams(x=x.data_ptr(), ldx=x.stride(0), ids=ids.data_ptr(), T=T, top_k=k, H=H, I=I,
                               expert_offset=experts.expert_offset, num_local=experts.num_experts,
                               w13=experts.w13.data_ptr(), s13=experts.s13.data_ptr(), g13=experts.g13.data_ptr(),
                               sw13=N.ptr(shared.w13) if shared else 0, ss13=N.ptr(shared.s13) if shared else 0,
                               sg13=N.ptr(shared.g13) if shared else 0, act=act.data_ptr())
        N.call("sl_moe_gate_up", C.byref(gp), N.stream())
        out = torch.empty(T, H, dtype=torch.float32, device=x.device)
        dp = N.MoeDownParams(act=act.data_ptr(), ids=ids.data_ptr(), wts=wts.data_ptr(), T=T, top_k=k, H=H, I=I,
                             expert_offset=experts.expert_offset, num_local=experts.num_experts,
                             w2=experts.w2.data_ptr(), s2=experts.s2.data_ptr(), g2=experts.g2.data_ptr(),
                             sw2=N.ptr(shared.w2) if shared else 0, ss2=N.ptr(shared.s2) if shared else 0,
                             sg2=N.ptr(shared.g2) if shared else 0, out=out.data_ptr(), out_f32=1, accumulate=0)
        if sink is not None:
            sink.pushed_rows = T
            N.call("sl_moe_down_push", C.byref(dp), C.byref(sink.push), N.stream())
            return sink
        N.call("sl_moe_down", C.byref(dp), N.stream())
        return out

    def _moe_grouped(self, x, experts, shared, ids, wts, sink=None, router=None):
        """Tensor-core weight streaming: routes that share an expert form one work item, so each
        chosen expert's weights are read once per step.  With `router` (a layer's weights) the
        router product, the routing and the plan run in the first kernel and ids/wts are outputs."""
        T, H = x.shape
        dev = x.device
        c = self.cfg
        rargs = None
        if router is not None:
            k = c.num_experts_per_tok
            E = router.router_w.shape[0]
            ids = torch.empty(T, k, dtype=torch.int32, device=dev)
            wts = torch.empty(T, k, dtype=torch.float32, device=dev)
            slabs = torch.empty(T, E, dtype=torch.float32, device=dev)          # the router's logits
            counter = self._zero_counter(dev)
            rargs = N.MoeRouterArgs(router_w=router.router_w.data_ptr(), bias=N.ptr(router.router_bias), E=E,
                                    n_group=c.n_group, topk_group=c.topk_group, norm=int(c.norm_topk_prob),
                                    scale=float(c.routed_scaling_factor), slabs=slabs.data_ptr(), counter=counter.data_ptr())
        k = ids.shape[1]
        I = experts.inter
        routes = T * k + (T if shared is not None else 0)
        max_items = T * k + (T + 7) // 8
        if self._persist_moe and (shared is None or shared.inter == I) and N.fn("sl_moe_persist_ok")(
                T, k, H, I, router.router_w.shape[0] if router is not None else 0, experts.num_experts,
                int(router is not None)):
            return self._moe_persist(x, experts, shared, ids, wts, sink, router, routes, max_items)
        xp = self._perm_of(x, T, H)
        xp_ready = xp is not None
        if not xp_ready:
            xp = torch.empty(((T + 7) // 8) * 8 * H, dtype=torch.float16, device=dev)
        act = torch.empty((routes + 8) * I, dtype=torch.float16, device=dev)
        y_route = torch.empty(routes, H, dtype=torch.float32, device=dev)
        plan = torch.empty(max_items * 9 + 1, dtype=torch.int32, device=dev)
        out = None if sink is not None else torch.empty(T, H, dtype=torch.float32, device=dev)
        a = N.MoeGroupedArgs(x=x.data_ptr(), ldx=x.stride(0), ids=ids.data_ptr(), wts=wts.data_ptr(), T=T, top_k=k, H=H, I=I,
                             expert_offset=experts.expert_offset, num_local=experts.num_experts,
                             w13=experts.w13.data_ptr(), s13=experts.s13.data_ptr(), g13=experts.g13.data_ptr(),
                             sw13=N.ptr(shared.w13) if shared else 0, ss13=N.ptr(shared.s13) if shared else 0,
                             sg13=N.ptr(shared.g13) if shared else 0,
                             w2=experts.w2.data_ptr(), s2=experts.s2.data_ptr(), g2=experts.g2.data_ptr(),
                             sw2=N.ptr(shared.w2) if shared else 0, ss2=N.ptr(shared.s2) if shared else 0,
                             sg2=N.ptr(shared.g2) if shared else 0,
                             xp=xp.data_ptr(), act_perm=act.data_ptr(), y_route=y_route.data_ptr(), plan=plan.data_ptr(),
                             max_items=max_items, out=N.ptr(out), xp_ready=int(xp_ready))
        if sink is not None:
            sink.pushed_rows = T
            N.call("sl_moe_grouped_mma", C.byref(a), C.cast(C.byref(rargs), C.c_void_p) if rargs is not None else None,
                   C.cast(C.byref(sink.push), C.c_void_p), N.stream())
            return sink
        N.call("sl_moe_grouped_mma", C.byref(a), C.cast(C.byref(rargs), C.c_void_p) if rargs is not None else None, None,
               N.stream())
        return out

    def _moe_persist(self, x, experts, shared, ids, wts, sink, router, routes, max_items):
        """The whole decode MoE layer in one persistent kernel (`csrc/moe_persist.cu`): router tiles, plan, gate/up, down and
        the weighted sum are tiles of one ordered queue with completion counters instead of five launches."""
        T, H = x.shape
        dev = x.device
        c = self.cfg
        k, I = ids.shape[1], experts.inter
        xp = self._perm_of(x, T, H)
        if xp is None:
            xp = torch.empty(((T + 7) // 8) * 8 * H, dtype=torch.float16, device=dev)
            N.call("sl_permute_x", xp.data_ptr(), x.data_ptr(), T, H, x.stride(0), N.stream())
        E = router.router_w.shape[0] if router is not None else 0
        slabs = torch.empty(4 * T * max(E, 1), dtype=torch.float32, device=dev)
        act = torch.empty((routes + 8) * I, dtype=torch.float16, device=dev)
        y_route = torch.empty(routes, H, dtype=torch.float32, device=dev)
        plan = torch.empty(max_items * 9 + 1, dtype=torch.int32, device=dev)
        out = None if sink is not None else torch.empty(T, H, dtype=torch.float32, device=dev)
        sync = self._persist_sync(dev)
        a = N.MoePersistArgs(
            x=x.data_ptr(), ldx=x.stride(0), xp=xp.data_ptr(), router_w=N.ptr(router.router_w) if router is not None else 0,
            bias=N.ptr(router.router_bias) if router is not None else 0, E=E, n_group=c.n_group, topk_group=c.topk_group,
            norm=int(c.norm_topk_prob), scale=float(c.routed_scaling_factor), T=T, top_k=k, H=H, I=I,
            expert_offset=experts.expert_offset, num_local=experts.num_experts,
            w13=experts.w13.data_ptr(), s13=experts.s13.data_ptr(), g13=experts.g13.data_ptr(),
            sw13=N.ptr(shared.w13) if shared else 0, ss13=N.ptr(shared.s13) if shared else 0, sg13=N.ptr(shared.g13) if shared else 0,
            w2=experts.w2.data_ptr(), s2=experts.s2.data_ptr(), g2=experts.g2.data_ptr(),
            sw2=N.ptr(shared.w2) if shared else 0, ss2=N.ptr(shared.s2) if shared else 0, sg2=N.ptr(shared.g2) if shared else 0,
            slabs=slabs.data_ptr(), act_perm=act.data_ptr(), y_route=y_route.data_ptr(), plan=plan.data_ptr(),
            ids=ids.data_ptr(), wts=wts.data_ptr(), sync=sync.data_ptr(), status=self._guard(dev) + 16,
            out=N.ptr(out), max_items=max_items, gsub=self._persist_gsub, trace=N.ptr(self._persist_trace))
        if sink is not None:
            sink.pushed_rows = T
            N.call("sl_moe_persist", C.byref(a), C.cast(C.byref(sink.push), C.c_void_p), N.stream())
            return sink
        N.call("sl_moe_persist", C.byref(a), None, N.stream())
        return out

    PERSIST_SYNC_WORDS = 512          # tile queue + completion counters of the persistent kernels (zero between launches)

    def _persist_sync(self, dev) -> torch.Tensor:
        key = ("persist", dev.type, dev.index)
        t = self._counters.get(key)
        if t is None:
            from . import tcgen05
            t = torch.zeros(self.PERSIST_SYNC_WORDS, dtype=torch.int32, device=dev)
            self._counters[key] = t
            tcgen05.on_error_reset(dev, t.zero_)        # a kernel that gave up leaves its counters as they were
        return t

    def check_persistent_status(self) -> None:
        """Raise if a kernel recorded an expired wait or a failed self-check since the last call (status words 8..11 of the
        device's error block belong to the persistent kernels)."""
        from . import tcgen05
        for key in list(self._counters):
            if isinstance(key, tuple) and key[0] == "persist":
                tcgen05.check_errors(torch.device(key[1], key[2]))

    @staticmethod
    def _guard(dev) -> int:
        """Address of the per-device index self-check record (words 4..7 of the error block)."""
        from . import tcgen05
        return tcgen05.error_flag(dev).data_ptr() + 16

    def _zero_counter(self, dev):
        """A device word that the fused router kernel expects to be zero and leaves zero."""
        key = (dev.type, dev.index)
        t = self._counters.get(key)
        if t is None:
            t = torch.zeros(1, dtype=torch.int32, device=dev)
            self._counters[key] = t
        return t

    def _route_fused(self, x, lw):
        """(ids, wts) of up to 32 token rows from the fused router kernel alone (router product + grouped top-k in one
        launch); falls back to the two-launch `route` for shapes that kernel does not take."""
        T, H = x.shape
        c = self.cfg
        k, E = c.num_experts_per_tok, lw.router_w.shape[0]
        if not (T <= DECODE_MAX_T and H % 256 == 0 and E <= 512 and x.stride(-1) == 1 and x.stride(0) % 8 == 0
                and lw.router_w.dtype == torch.bfloat16 and T * k <= 480):
            return self.route(x, lw)
        dev = x.device
        ids = torch.empty(T, k, dtype=torch.int32, device=dev)
        wts = torch.empty(T, k, dtype=torch.float32, device=dev)
        logits = torch.empty(T, E, dtype=torch.float32, device=dev)
        max_items = T * k + (T + 7) // 8
        plan = torch.empty(max_items * 9 + 1, dtype=torch.int32, device=dev)
        rargs = N.MoeRouterArgs(router_w=lw.router_w.data_ptr(), bias=N.ptr(lw.router_bias), E=E, n_group=c.n_group,
                                topk_group=c.topk_group, norm=int(c.norm_topk_prob), scale=float(c.routed_scaling_factor),
                                slabs=logits.data_ptr(), counter=self._zero_counter(dev).data_ptr())
        a = N.MoeGroupedArgs(x=x.data_ptr(), ldx=x.stride(0), ids=ids.data_ptr(), wts=wts.data_ptr(), T=T, top_k=k, H=H,
                             I=lw.experts.inter, expert_offset=lw.experts.expert_offset, num_local=lw.experts.num_experts,
                             plan=plan.data_ptr(), max_items=max_items, xp_ready=1)
        try:
            N.call("sl_moe_grouped_mma", C.byref(a), C.byref(rargs), None, N.stream())
        except N.NativeError:
            return self.route(x, lw)
        return ids, wts

    # -- decode MoE on the block-scaled FP4 tensor-core GEMMs -----------------------------------------------------
    FP4_DECODE_MIN_WORK = 16384       # token rows x expert intermediate size from which the FP4 form streams faster

    def _fp4_decode_ok(self, T: int, lw) -> bool:
        """The weight-streaming kernels expand FP4 -> f16 on the CUDA cores, which bounds them near 3.3 TB/s of weights
        per GPU; the tcgen05 kind::mxf4nvf4 GEMMs read the packed weights at the HBM rate but cost six launches and 4-bit
        activations.  They win once the step streams enough bytes per expert (whole layer in a CUDA graph, streaming ->
        FP4): TP 1: 356 -> 303 us at 8 rows, 635 -> 481 at 16, 1011 -> 717 at 32; TP 2: equal at 8, 350 -> 285 at 16,
        543 -> 417 at 32; TP 4: 303 -> 289 at 32 and behind below; TP 8: behind at every size (187 vs 246 us at 32 rows).
        SLOPLLM_B200_MOE_FP4_DECODE=0 / 1 forces the choice."""
        from . import gemm
        ex = lw.experts
        if T < 2 or T > DECODE_MAX_T or not gemm.fp4_moe_ok(ex, self.cfg.hidden_size):
            return False
        if lw.shared is not None and (lw.shared.inter != ex.inter or not lw.shared.is_nvfp4):
            return False
        if T * self.cfg.num_experts_per_tok > 512 or ex.num_experts > 1024:
            return False
        force = self._fp4_decode_force
        if force in ("0", "1"):
            return force == "1"
        return T * ex.inter >= self.FP4_DECODE_MIN_WORK

    def _moe_fp4_decode(self, x, lw, ids, wts, sink=None):
        """Expert MLP of a few token rows on `tcgen05.mma.kind::mxf4nvf4` (W4A4): the token rows are quantised once and are
        the narrow operand of EVERY expert tile of the gate/up GEMM, whose epilogue keeps the tokens routed to that expert;
        the activations land in 32-row blocks per touched expert, are quantised, and the down GEMM's epilogue scatters its
        columns to per-route rows, which the weighted reduce (+ push) sums.  No sort, no gather."""
        from . import fp4, gemm, tcgen05
        ex, sh = lw.experts, lw.shared
        T, H = x.shape
        k = ids.shape[1]
        I, E = ex.inter, ex.num_experts
        dev = x.device
        sf13, sf2 = gemm._sf_tiles_of(ex)
        ssf13, ssf2 = gemm._sf_tiles_of(sh) if sh is not None else (None, None)
        max_slots = min(E, T * k)
        rows = (max_slots + 1) * 32
        tb = N.kernels().sl_fp4_tile_bytes()
        mt1, mt2 = (max_slots + 1) * (I // 128), (max_slots + 1) * (H // 128)
        tiles1 = torch.empty(mt1 * tb, dtype=torch.uint8, device=dev)
        tiles2 = torch.empty(mt2 * tb, dtype=torch.uint8, device=dev)
        meta = torch.empty(3, dtype=torch.int32, device=dev)                  # tiles of each GEMM, activation rows in use
        tab1 = torch.empty(rows, dtype=torch.int32, device=dev)
        tab2 = torch.empty(rows, dtype=torch.int32, device=dev)
        ids = ids.to(torch.int32).contiguous()
        N.call("sl_fp4_decode_plan", ids.data_ptr(), T, k, ex.expert_offset, E, int(sh is not None), I, H, tiles1.data_ptr(),
               meta.data_ptr(), tiles2.data_ptr(), meta.data_ptr() + 4, tab1.data_ptr(), tab2.data_ptr(), meta.data_ptr() + 8,
               max_slots, N.stream())
        xq, sfx, gx = fp4.quantize_rows(self._bf16(x), bn=32)
        err = tcgen05.error_flag(dev).data_ptr()
        act = torch.empty(rows, I, dtype=torch.bfloat16, device=dev)
        g13 = ex.g13.to(torch.float32).contiguous()
        N.call("sl_gemm_fp4_tcgen05_tab", ex.w13.data_ptr(), sf13.data_ptr(), g13.data_ptr(), E * 2 * I,
               N.ptr(sh.w13) if sh is not None else 0, N.ptr(ssf13), N.ptr(sh.g13) if sh is not None else 0, 2 * I,
               xq.data_ptr(), sfx.data_ptr(), gx.data_ptr(), T, act.data_ptr(), I, 0, tab1.data_ptr(), H, I, 32,
               tiles1.data_ptr(), meta.data_ptr(), mt1, err, N.stream())
        aq, sfa, ga = fp4.quantize_rows(act, bn=32, num_rows=meta[2:3])
        routes = T * k + (T if sh is not None else 0)
        y_route = torch.empty(routes, H, dtype=torch.float32, device=dev)
        g2 = ex.g2.to(torch.float32).contiguous()
        N.call("sl_gemm_fp4_tcgen05_tab", ex.w2.data_ptr(), sf2.data_ptr(), g2.data_ptr(), E * H,
               N.ptr(sh.w2) if sh is not None else 0, N.ptr(ssf2), N.ptr(sh.g2) if sh is not None else 0, H,
               aq.data_ptr(), sfa.data_ptr(), ga.data_ptr(), rows, y_route.data_ptr(), H, 1, tab2.data_ptr(), I, 0, 32,
               tiles2.data_ptr(), meta.data_ptr() + 4, mt2, err, N.stream())
        wts = wts.to(torch.float32).contiguous()
        if sink is not None:
            sink.pushed_rows = T
            N.call("sl_moe_route_reduce", y_route.data_ptr(), ids.data_ptr(), wts.data_ptr(), T, k, H, ex.expert_offset, E,
                   int(sh is not None), 0, C.byref(sink.push), N.stream())
            return sink
        out = torch.empty(T, H, dtype=torch.float32, device=dev)
        N.call("sl_moe_route_reduce", y_route.data_ptr(), ids.data_ptr(), wts.data_ptr(), T, k, H, ex.expert_offset, E,
               int(sh is not None), out.data_ptr(), 0, N.stream())
        return out

    def moe_tp(self, x, lw, sink=None):
        T, H = x.shape
        if (x.is_cuda and lw.experts.is_nvfp4 and lw.router_w.dtype == torch.bfloat16 and not self._persist_moe
                and self._fp4_decode_ok(T, lw)):
            x = self._bf16(x)
            ids, wts = self._route_fused(x, lw)
            return self._moe_fp4_decode(x, lw, ids, wts, sink)
        fused_ok = (T <= DECODE_MAX_T and lw.experts.is_nvfp4 and H % 256 == 0 and lw.experts.inter % 128 == 0
                    and T * self.cfg.num_experts_per_tok <= 480 and lw.router_w.dtype == torch.bfloat16
                    and (lw.shared is None or lw.shared.inter == lw.experts.inter))
        if fused_ok:
            x = self._bf16(x)
            if x.stride(-1) == 1 and x.stride(0) % 8 == 0:
                return self._moe_grouped(x, lw.experts, lw.shared, None, None, sink, router=lw)
        ids, wts = self.route(x, lw)
        if x.shape[0] <= DECODE_MAX_T and lw.experts.is_nvfp4:
            if lw.shared is not None and lw.shared.inter != lw.experts.inter:
                out = self._moe_small(x, lw.experts, None, ids, wts) + self.shared_expert(x, lw)
                return out if sink is None else sink.push_tensor(out)
            return self._moe_small(x, lw.experts, lw.shared, ids, wts, sink)
        from .gemm import moe_large
        out = moe_large(self, x, lw.experts, lw.shared, ids, wts)
        return out if sink is None else sink.push_tensor(out)

    def moe_local_experts(self, x, experts, ids, w):
        ids = ids.to(torch.int32).contiguous()
        w = w.to(torch.float32).contiguous()
        if x.shape[0] <= DECODE_MAX_T and experts.is_nvfp4:
            return self._moe_small(x, experts, None, ids, w)
        from .gemm import moe_large
        return moe_large(self, x, experts, None, ids, w)

    def shared_expert(self, x, lw):
        T = x.shape[0]
        ids = torch.zeros(T, 1, dtype=torch.int32, device=x.device)
        w = torch.ones(T, 1, dtype=torch.float32, device=x.device)
        if T <= DECODE_MAX_T and lw.shared.is_nvfp4:
            return self._moe_small(x, lw.shared, None, ids, w)
        from .gemm import moe_large
        return moe_large(self, x, lw.shared, None, ids, w)

    # -- head ----------------------------------------------------------------------------------------
    def logits(self, x, lm_head):
        return self.linear(x, lm_head, out_f32=True)

    def argmax(self, logits, id_offset: int = 0, want_val: bool = False):
        B, V = logits.shape
        out = torch.empty(B, dtype=torch.int64, device=logits.device)
        val = torch.empty(B, dtype=torch.float32, device=logits.device) if want_val else None
        sv = torch.empty(B, 64, dtype=torch.float32, device=logits.device)
        si = torch.empty(B, 64, dtype=torch.int32, device=logits.device)
        N.call("sl_argmax", out.data_ptr(), logits.data_ptr(), B, V, logits.stride(0), int(logits.dtype == torch.float32),
               id_offset, N.ptr(val), sv.data_ptr(), si.data_ptr(), N.stream())
        return (out, val) if want_val else out


_ = Optional
