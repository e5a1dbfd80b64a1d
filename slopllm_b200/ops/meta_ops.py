"""Shape-only backend: every staged op returns `meta` tensors of the right shape and dtype and
records its bytes / FLOPs, without touching a device.  Used to size a deployment (activation
memory per step, weight bytes streamed per decode step, FLOPs per prefill chunk) and to test the
model's shape plumbing for configurations that do not fit the test machine.

Reference: `src/meta_ops.ts:1-549` (MetaOps, the fake `DeviceOps`).
"""
from __future__ import annotations

from collections import defaultdict

import torch


def _meta(*shape, dtype=torch.bfloat16):
    return torch.empty(*shape, dtype=dtype, device="meta")


class MetaOps:
    name = "meta"
    act_dtype = torch.bfloat16

    def __init__(self, cfg, ctx=None):
        self.cfg = cfg
        self.ctx = ctx
        self.flops = defaultdict(float)           # op name -> multiply-add FLOPs (2 per MAC)
        self.weight_bytes = defaultdict(float)    # op name -> bytes of weights the op reads
        self.calls = defaultdict(int)

    def _note(self, op: str, flops: float = 0.0, wbytes: float = 0.0) -> None:
        self.calls[op] += 1
        self.flops[op] += flops
        self.weight_bytes[op] += wbytes

    @staticmethod
    def _wbytes(w) -> float:
        n = w.weight.numel() * w.weight.element_size()
        if getattr(w, "scale", None) is not None:
            n += w.scale.numel() * w.scale.element_size()
        return float(n)

    # -- elementwise / linear ---------------------------------------------------------------------------
    def embed(self, ids, table):
        self._note("embed")
        return _meta(ids.shape[0], table.shape[1])

    def rmsnorm(self, x, w, eps=None):
        self._note("rmsnorm")
        return _meta(*x.shape)

    def add_rmsnorm(self, x, residual, w, eps=None, want_perm: bool = False):
        self._note("add_rmsnorm")
        return _meta(*x.shape), _meta(*x.shape, dtype=torch.float32)

    def linear(self, x, w, out_f32: bool = False, sink=None, defer_reduce: bool = False):
        T = x.shape[0]
        self._note("linear", 2.0 * T * w.in_features * w.out_features, self._wbytes(w))
        return _meta(T, w.out_features, dtype=torch.float32 if out_f32 else torch.bfloat16)

    # -- attention ------------------------------------------------------------------------------------------
    def attn_pre(self, qkv, lw, st, layer_cache):
        c, T = self.cfg, qkv.shape[0]
        self._note("attn_pre")
        return _meta(T, c.q_lora_rank), (_meta(T, c.index_n_heads, dtype=torch.float32) if lw.has_indexer else None)

    def q_post(self, qb, lw, st, idx_w):
        c, T, hl = self.cfg, qb.shape[0], lw.w_kn.shape[0]
        self._note("q_post", 2.0 * T * hl * c.qk_nope_head_dim * c.kv_lora_rank, float(lw.w_kn.numel() * 2))
        q8 = w_eff = None
        if lw.has_indexer:
            q8 = _meta(T, c.index_n_heads, c.index_head_dim, dtype=torch.uint8)
            w_eff = _meta(T, c.index_n_heads, dtype=torch.float32)
        return _meta(T, hl, c.kv_lora_rank), _meta(T, hl, c.qk_rope_head_dim), q8, w_eff

    def indexer_topk(self, q8, w_eff, layer_cache, st):
        c, T = self.cfg, q8.shape[0]
        keys = -(-max(1, st.max_kv_len) // max(1, st.cp_world))
        self._note("indexer_topk", 2.0 * T * keys * c.index_n_heads * c.index_head_dim)
        return _meta(T, c.index_topk, dtype=torch.int32), _meta(T, c.index_topk, dtype=torch.float32)

    def topk_to_slots(self, topk_pos, st, local_only: bool = False):
        self._note("topk_to_slots")
        return _meta(*topk_pos.shape, dtype=torch.int32), _meta(topk_pos.shape[0], dtype=torch.int32)

    def sparse_mla(self, q_abs, q_pe, layer_cache, slots, lengths):
        c = self.cfg
        T, h, R = q_abs.shape
        keys = min(slots.shape[1], max(1, -(-c.index_topk // 1)))
        self._note("sparse_mla", 2.0 * T * h * keys * (2 * R + c.qk_rope_head_dim))
        return _meta(T, h, R), _meta(T, h, dtype=torch.float32)

    def v_expand(self, o, w_v):
        T, hl, R = o.shape
        self._note("v_expand", 2.0 * T * hl * R * w_v.shape[2], float(w_v.numel() * 2))
        return _meta(T, hl * w_v.shape[2])

    def merge_attention_partials(self, o, lse):
        return _meta(*o.shape[1:]), _meta(*lse.shape[1:], dtype=torch.float32)

    # -- MLP ------------------------------------------------------------------------------------------------
    def dense_mlp(self, x, lw, sink=None):
        T = x.shape[0]
        for w in (lw.mlp_w13, lw.mlp_w2):
            self._note("dense_mlp", 2.0 * T * w.in_features * w.out_features, self._wbytes(w))
        return _meta(T, lw.mlp_w2.out_features, dtype=torch.float32)

    def route(self, x, lw):
        c, T = self.cfg, x.shape[0]
        self._note("route", 2.0 * T * lw.router_w.shape[0] * lw.router_w.shape[1], float(lw.router_w.numel() * 2))
        return _meta(T, c.num_experts_per_tok, dtype=torch.int32), _meta(T, c.num_experts_per_tok, dtype=torch.float32)

    def _expert_cost(self, T, experts, active_per_token):
        H, I = experts.hidden, experts.inter
        per_expert_bytes = 3.0 * H * I * (0.5 + 1.0 / 16 if experts.is_nvfp4 else 2.0)
        touched = min(experts.num_experts, T * active_per_token)
        return 2.0 * T * active_per_token * 3 * H * I, touched * per_expert_bytes

    def moe_tp(self, x, lw, sink=None):
        T = x.shape[0]
        self.route(x, lw)
        f, b = self._expert_cost(T, lw.experts, self.cfg.num_experts_per_tok)
        if lw.shared is not None:
            f2, b2 = self._expert_cost(T, lw.shared, 1)
            f, b = f + f2, b + b2
        self._note("moe", f, b)
        return _meta(T, x.shape[1], dtype=torch.float32)

    def moe_local_experts(self, x, experts, ids, w):
        f, b = self._expert_cost(x.shape[0], experts, ids.shape[1])
        self._note("moe", f, b)
        return _meta(x.shape[0], x.shape[1], dtype=torch.float32)

    def shared_expert(self, x, lw):
        f, b = self._expert_cost(x.shape[0], lw.shared, 1)
        self._note("moe", f, b)
        return _meta(x.shape[0], x.shape[1], dtype=torch.float32)

    # -- head ------------------------------------------------------------------------------------------------
    def logits(self, x, lm_head):
        self._note("logits", 2.0 * x.shape[0] * lm_head.in_features * lm_head.out_features, self._wbytes(lm_head))
        return _meta(x.shape[0], lm_head.out_features, dtype=torch.float32)

    def argmax(self, logits, id_offset: int = 0, want_val: bool = False):
        return _meta(logits.shape[0], dtype=torch.int64)

    # -- report ------------------------------------------------------------------------------------------------
    def summary(self) -> dict:
        return {"flops": dict(self.flops), "weight_bytes": dict(self.weight_bytes), "calls": dict(self.calls),
                "total_flops": sum(self.flops.values()), "total_weight_bytes": sum(self.weight_bytes.values())}
