"""Op sets.

The model is written once against a small staged op interface; two op sets implement it:

* :class:`RefOps` — plain PyTorch fp32 (CPU plumbing model, and the oracle for tests);
* :class:`slopllm_b200.ops.cuda_ops.CudaOps` — hand-written sm_100a kernels (bf16 / NVFP4 /
  FP8), required on a GPU: it raises if the native library is missing.

`get_ops(device)` picks by device type.  The reference achieves the same "write the model
once" property with its `DeviceOps` interface (`src/device_ops.ts:40-229`) implemented by
`GlmOps`, `ParallelOps` and `MetaOps`.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import quant, reference as R


class RefOps:
    """fp32 PyTorch implementation of the staged model ops."""

    name = "reference"
    act_dtype = torch.float32

    def __init__(self, cfg, ctx=None):
        self.cfg = cfg
        self.ctx = ctx

    # -- elementwise / linear -------------------------------------------------------------
    def embed(self, ids, table):
        return table[ids.to(torch.int64)].to(torch.float32)

    def rmsnorm(self, x, w, eps=None):
        return R.rmsnorm(x, w, self.cfg.rms_norm_eps if eps is None else eps)

    def add_rmsnorm(self, x, residual, w, eps=None, want_perm: bool = False):
        return R.add_rmsnorm(x, residual, w, self.cfg.rms_norm_eps if eps is None else eps)

    def linear(self, x, w, out_f32: bool = False, sink=None, defer_reduce: bool = False):
        return R.linear(x, w)

    def merge_attention_partials(self, o, lse):
        return R.merge_attention_partials(o, lse)

    # -- attention stages -------------------------------------------------------------------
    def attn_pre(self, qkv, lw, st, layer_cache):
        """After the fused q_a|ckv|k_pe|(idx) projection: norms, rope, quantise, cache append.

        Returns (c_q [T, q_lora], idx_w [T, Hi] or None).
        """
        c = self.cfg
        q0, q1, q2 = c.q_lora_rank, c.q_lora_rank + c.kv_lora_rank, c.q_lora_rank + c.kv_lora_rank + c.qk_rope_head_dim
        cq = R.rmsnorm(qkv[:, :q0], lw.q_a_norm, c.rms_norm_eps)
        ckv = R.rmsnorm(qkv[:, q0:q1], lw.kv_a_norm, c.rms_norm_eps)
        kpe = R.apply_rope(qkv[:, q1:q2], st.positions, c.rope_theta, c.qk_rope_head_dim, c.rope_interleave)
        slots, owned = R.token_slots(st.page_table, st.batch_idx, st.positions, st.page_size, st.cp_world, st.cp_rank)
        R.kv_append(layer_cache.kv, quant.pack_kv_rows(ckv, kpe, c.kv_quant_group), slots, owned)
        idx_w = None
        if lw.has_indexer:
            q3 = q2 + c.index_head_dim
            k = R.layernorm(qkv[:, q2:q3], lw.idx_k_norm_w, lw.idx_k_norm_b)
            k = R.apply_rope(k, st.positions, c.rope_theta, c.qk_rope_head_dim, c.indexer_rope_interleave)
            R.kv_append(layer_cache.idx, quant.pack_index_rows(k), slots, owned)
            idx_w = qkv[:, q3:q3 + c.index_n_heads].to(torch.float32) * (c.index_n_heads ** -0.5)
        return cq, idx_w

    def q_post(self, qb, lw, st, idx_w):
        """After the q_b | (indexer wq_b) projection: rope, absorb, indexer-Q quantise.

        Returns (q_abs [T, hl, R], q_pe [T, hl, Dr], q8 [T, Hi, Di] or None, w_eff or None).
        """
        c = self.cfg
        T = qb.shape[0]
        hl = lw.w_kn.shape[0]
        dqk = c.qk_head_dim
        q = qb[:, :hl * dqk].reshape(T, hl, dqk)
        q_pe = R.apply_rope(q[..., c.qk_nope_head_dim:], st.positions, c.rope_theta, c.qk_rope_head_dim, c.rope_interleave)
        q_abs = R.absorb_q(q[..., :c.qk_nope_head_dim], lw.w_kn)
        q8 = w_eff = None
        if lw.has_indexer:
            qi = qb[:, hl * dqk:].reshape(T, c.index_n_heads, c.index_head_dim)
            qi = R.apply_rope(qi, st.positions, c.rope_theta, c.qk_rope_head_dim, c.indexer_rope_interleave)
            q8, w_eff = R.indexer_quantize_q(qi, idx_w, c.index_head_dim ** -0.5)
        return q_abs, q_pe, q8, w_eff

    def indexer_topk(self, q8, w_eff, layer_cache, st):
        c = self.cfg
        return R.indexer_topk(q8, w_eff, layer_cache.idx, st.page_table, st.batch_idx, st.positions, c.index_topk,
                              st.page_size, c.index_head_dim, st.cp_world, st.cp_rank)

    def topk_to_slots(self, topk_pos, st, local_only: bool = False):
        """Global positions -> this rank's slots.  With CP, `local_only` drops positions
        owned by other ranks before compaction."""
        if local_only and st.cp_world > 1:
            mine = (topk_pos >= 0) & ((topk_pos % st.cp_world) == st.cp_rank)
            topk_pos = torch.where(mine, topk_pos, torch.full_like(topk_pos, -1))
        return R.topk_to_slots(topk_pos, st.page_table, st.batch_idx, st.page_size, st.cp_world)

    def sparse_mla(self, q_abs, q_pe, layer_cache, slots, lengths):
        c = self.cfg
        return R.sparse_mla(q_abs, q_pe, layer_cache.kv, slots, lengths, c.softmax_scale, c.kv_lora_rank,
                            c.qk_rope_head_dim, c.kv_quant_group)

    def v_expand(self, o, w_v):
        return R.v_expand(o, w_v)

    # -- MLP ------------------------------------------------------------------------------------
    def dense_mlp(self, x, lw, sink=None):
        return R.linear(R.silu_mul(R.linear(x, lw.mlp_w13)), lw.mlp_w2)

    def route(self, x, lw):
        c = self.cfg
        logits = x.to(torch.float32) @ lw.router_w.to(torch.float32).t()
        return R.moe_route(logits, lw.router_bias, c.num_experts_per_tok, c.n_group, c.topk_group,
                           c.norm_topk_prob, c.routed_scaling_factor)

    def moe_tp(self, x, lw, sink=None):
        """TP-sliced experts: every rank holds all experts' I/W slice; returns the partial sum
        (routed + shared) that the next all-reduce completes."""
        ids, w = self.route(x, lw)
        out = R.moe_experts(x, lw.experts, ids, w)
        if lw.shared is not None:
            T = x.shape[0]
            out = out + R.moe_experts(x, lw.shared, torch.zeros(T, 1, dtype=torch.int32, device=x.device),
                                      torch.ones(T, 1, device=x.device))
        return out

    def moe_local_experts(self, x, experts, ids, w):
        """Experts held by this rank only (EP): ids are global; rows whose expert lives
        elsewhere contribute nothing."""
        lo, hi = experts.expert_offset, experts.expert_offset + experts.num_experts
        mine = (ids >= lo) & (ids < hi)
        w = torch.where(mine, w, torch.zeros_like(w))
        ids = torch.where(mine, ids, torch.full_like(ids, lo))
        return R.moe_experts(x, experts, ids, w)

    def shared_expert(self, x, lw):
        T = x.shape[0]
        return R.moe_experts(x, lw.shared, torch.zeros(T, 1, dtype=torch.int32, device=x.device),
                             torch.ones(T, 1, device=x.device))

    # -- head -------------------------------------------------------------------------------------
    def logits(self, x, lm_head):
        return R.linear(x, lm_head)

    def argmax(self, logits):
        return logits.argmax(-1)


def get_ops(cfg, device, ctx=None):
    device = torch.device(device)
    if device.type == "cuda":
        from .cuda_ops import CudaOps
        return CudaOps(cfg, ctx)
    return RefOps(cfg, ctx)


__all__ = ["RefOps", "get_ops", "quant", "R"]
_ = Optional
