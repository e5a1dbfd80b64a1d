"""Memory plan of a deployment (glm_moe_dsa, and the dense Qwen3 / Qwen3.5 families), computed from the configuration alone
(no weights, no GPU).

`plan_memory` answers the questions that come before a launch: how many bytes of weights does one rank hold under a given
tensor / expert / context parallelism, what does one KV page cost, how many pages fit next to the weights in the device
memory that `--arena` allows, and how much context that is.  The reference answers them with its shape-only backend
(`src/meta_ops.ts`) and the sizing notes in `GLM51-NVFP4-weights.md`; here the same arithmetic is a function and a command
(`python -m slopllm_b200 plan`).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Dict

from ..config import PAGE_SIZE, GlmMoeDsaConfig

GIB = 1 << 30


def _lin(n: int, k: int, nvfp4: bool, elem: int = 2) -> int:
    """Bytes of an [n, k] linear weight: NVFP4 = half a byte per weight + one e4m3 scale per 16 + one fp32 global."""
    return n * k // 2 + n * k // 16 + 4 if nvfp4 else n * k * elem


def layer_weight_bytes(cfg: GlmMoeDsaConfig, layer: int, tp: int = 1, ep: bool = False, elem: int = 2) -> int:
    """Bytes of one decoder layer on one rank: attention projections head-sharded, o_proj / down row-sharded, gate / up
    column-sharded, the small replicated projections and norms whole; with `ep` the routed experts are split by expert
    instead of by intermediate column (the shared expert stays column-sharded)."""
    H, R, Dr = cfg.hidden_size, cfg.kv_lora_rank, cfg.qk_rope_head_dim
    Dn, Dv, Q = cfg.qk_nope_head_dim, cfg.v_head_dim, cfg.q_lora_rank
    hl = cfg.num_attention_heads // tp
    full = cfg.indexer_is_full(min(layer, len(cfg.indexer_types) - 1)) if cfg.indexer_types else False
    Hi, Di = cfg.index_n_heads, cfg.index_head_dim
    qkv_rows = Q + R + Dr + ((Di + Hi) if full else 0)
    qb_rows = hl * (Dn + Dr) + (Hi * Di if full else 0)
    b = _lin(qkv_rows, H, False, elem) + _lin(qb_rows, Q, False, elem)
    b += hl * (Dn + Dv) * R * elem                                    # absorbed k_nope and v projections
    b += _lin(H, hl * Dv, bool(cfg.quant_o_proj), elem)
    b += (2 * H + Q + R + (2 * Di if full else 0)) * elem             # norms
    if cfg.is_moe_layer(layer):
        E, I = cfg.n_routed_experts, cfg.moe_intermediate_size
        q = bool(cfg.quant_experts)
        b += E * H * elem + E * 4                                     # router weight + bias
        if ep:
            b += (E // tp) * (_lin(2 * I, H, q, elem) + _lin(H, I, q, elem))
        else:
            b += E * (_lin(2 * I // tp, H, q, elem) + _lin(H, I // tp, q, elem))
        if cfg.n_shared_experts:
            Is = I * cfg.n_shared_experts // tp
            b += _lin(2 * Is, H, q, elem) + _lin(H, Is, q, elem)
    else:
        I = cfg.intermediate_size // tp
        q = bool(cfg.quant_dense_mlp)
        b += _lin(2 * I, H, q, elem) + _lin(H, I, q, elem)
    return b


def model_weight_bytes(cfg: GlmMoeDsaConfig, tp: int = 1, ep: bool = False, with_mtp: bool = True, elem: int = 2) -> int:
    H, V = cfg.hidden_size, cfg.vocab_size
    n = cfg.num_hidden_layers + (cfg.num_nextn_predict_layers if with_mtp else 0)
    b = V * H * elem + (V // tp) * H * elem + H * elem                # embedding (whole), lm_head shard, final norm
    for i in range(n):
        b += layer_weight_bytes(cfg, i, tp, ep, elem)
        if i >= cfg.num_hidden_layers:                                # MTP layer extras: two norms, eh_proj, head norm
            b += 3 * H * elem + _lin(H, 2 * H, False, elem)
    return b


def kv_page_bytes(cfg: GlmMoeDsaConfig, with_mtp: bool = True) -> int:
    """Bytes one page id costs on one rank: 64 rows per layer of the packed sparse-MLA cache, plus the indexer key rows
    of the layers that own an indexer.  Under context parallelism a page id covers 64 x W tokens and every rank stores 64
    of them, so this figure does not change with W; the tokens per page do."""
    n = cfg.num_hidden_layers + (cfg.num_nextn_predict_layers if with_mtp else 0)
    per_token = 0
    for i in range(n):
        per_token += cfg.kv_row_bytes
        if cfg.indexer_is_full(min(i, len(cfg.indexer_types) - 1)):
            per_token += cfg.index_row_bytes
    return per_token * PAGE_SIZE


def step_workspace_bytes(cfg: GlmMoeDsaConfig, tp: int, chunk: int, context: int, cp: int = 1) -> int:
    """Upper estimate of the transient buffers of one prefill chunk of `chunk` tokens against `context` cached tokens: the
    residual and activation rows, the expert-sorted MoE rows, the sparse-MLA query / output rows, and the indexer's score
    matrix (bounded by its 2 GiB budget)."""
    H, k = cfg.hidden_size, max(1, cfg.num_experts_per_tok)
    hl = max(1, cfg.num_attention_heads // tp) * (cp if cp > 1 else 1)     # CP gathers all heads
    I = max(cfg.moe_intermediate_size, 1) // tp
    act = chunk * H * (4 + 4 + 2 + 2)                                      # residual in / out (fp32), normed x, attention out
    moe = chunk * k * (H * 2 + 2 * I * 2 + I * 2 + H * 2) + chunk * H * 4  # sorted rows, gate/up, act, down rows, fp32 out
    mla = chunk * hl * (cfg.kv_lora_rank + cfg.qk_rope_head_dim) * 2 + chunk * hl * cfg.kv_lora_rank * 4 * 2
    keys = -(-context // max(1, cp))
    scores = min(chunk * keys * 4, 2 * GIB) + chunk * cfg.index_topk * 12
    dense = chunk * 2 * (cfg.intermediate_size // tp) * 2 * 2
    return act + max(moe, dense) + mla + scores


@dataclass
class MemoryPlan:
    tp: int
    cp: int
    ep: bool
    weights_bytes: int
    page_bytes: int
    tokens_per_page: int
    workspace_bytes: int
    budget_bytes: int
    max_pages: int
    max_tokens: int
    requested_pages: int
    requested_fits: bool

    def to_dict(self) -> Dict[str, object]:
        d = asdict(self)
        d.update(weights_gib=round(self.weights_bytes / GIB, 2), workspace_gib=round(self.workspace_bytes / GIB, 2),
                 kv_gib_at_max=round(self.max_pages * self.page_bytes / GIB, 2), budget_gib=round(self.budget_bytes / GIB, 2))
        return d


def plan_memory(cfg: GlmMoeDsaConfig, world: int = 1, cp: bool = False, ep: bool = False, mtp: int = 0, batch_size: int = 8,
                chunk_size: int = 8192, max_pages: int = 0, arena_gb: float = 0.0, device_gb: float = 180.0,
                context: int = 0, reserve_gb: float = 4.0) -> MemoryPlan:
    """The plan for one rank of a `world`-GPU replica.  `arena_gb` (0: `device_gb`) is what the process may allocate;
    `reserve_gb` stays free for the CUDA context, NCCL and the symmetric region.  `context` is the longest sequence the
    workspace estimate assumes (0: the pages asked for, or 64K tokens)."""
    tp = world
    cpw = world if cp else 1
    weights = model_weight_bytes(cfg, tp, ep, with_mtp=mtp > 0)
    page = kv_page_bytes(cfg, with_mtp=mtp > 0)
    tpp = PAGE_SIZE * cpw
    requested = max_pages if max_pages > 0 else batch_size * -(-chunk_size // PAGE_SIZE)
    ctx = context or (max_pages * tpp if max_pages > 0 else 65536)
    work = step_workspace_bytes(cfg, tp, chunk_size, ctx, cpw)
    budget = int(((arena_gb if arena_gb > 0 else device_gb) - reserve_gb) * GIB)
    left = budget - weights - work
    fit = max(0, left // page)
    return MemoryPlan(tp=tp, cp=cpw, ep=ep, weights_bytes=weights, page_bytes=page, tokens_per_page=tpp, workspace_bytes=work,
                      budget_bytes=budget, max_pages=int(fit), max_tokens=int(fit) * tpp, requested_pages=requested,
                      requested_fits=requested <= fit)


# ---- dense families (Qwen3, Qwen3.5) -----------------------------------------------------------------------------------

def dense_weight_bytes(cfg, tp: int = 1, elem: int = 2, fp8: bool = False) -> int:
    """Per-rank weight bytes of a Qwen3 / Qwen3.5 decoder: attention and Gated-DeltaNet projections head-sharded, MLP
    column / row sharded, embedding whole, lm_head vocabulary-sharded.  `fp8`: the attention and MLP projections stay FP8
    (one byte per weight + one fp32 scale per 128 x 128 block)."""
    H, I, hd = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim

    def lin(n, k, quant=False):
        return n * k + (-(-n // 128)) * (-(-k // 128)) * 4 if quant else n * k * elem
    b = cfg.vocab_size * H * elem + H * elem
    b += (cfg.vocab_size // tp) * H * elem                         # the head's shard is materialised even when it is tied
    for kind in cfg.layer_types:
        b += 2 * H * elem                                           # the two layer norms
        b += lin(2 * I // tp, H, fp8) + lin(H, I // tp, fp8)
        if kind == "full_attention":
            qs = hd * (2 if cfg.attn_output_gate else 1)
            hq, hk = cfg.num_attention_heads // tp, max(1, cfg.num_key_value_heads // tp)
            b += lin(hq * qs + 2 * hk * hd, H, fp8) + lin(H, hq * hd, fp8) + 2 * hd * elem      # qkv, o_proj, q/k norms
        else:
            lh, dk, dv = cfg.linear_num_key_heads // tp, cfg.linear_key_head_dim, cfg.linear_value_head_dim
            conv_dim = lh * (2 * dk + dv)
            b += lin(conv_dim + lh * dv + 2 * lh, H) + lin(H, lh * dv)                          # in-projection, out-projection
            b += conv_dim * cfg.linear_conv_kernel_dim * elem + 2 * lh * 4 + dv * elem          # conv, A_log, dt_bias, norm
    return b


def dense_kv_page_bytes(cfg, tp: int = 1, elem: int = 2) -> int:
    """Bytes of one 64-token page on one rank: K and V rows of every full-attention layer (recurrent layers keep their
    state per sequence, not per page)."""
    n_kv = max(1, cfg.num_key_value_heads // tp)
    full = sum(1 for k in cfg.layer_types if k == "full_attention")
    return full * 2 * n_kv * cfg.head_dim * elem * PAGE_SIZE


def plan_dense(cfg, world: int = 1, batch_size: int = 8, chunk_size: int = 8192, max_pages: int = 0, arena_gb: float = 0.0,
               device_gb: float = 180.0, fp8: bool = False, reserve_gb: float = 4.0) -> MemoryPlan:
    """`plan_memory` for the dense families (tensor parallel only; the workspace estimate is the residual / activation rows
    plus the MLP's gate-up rows of one chunk)."""
    weights = dense_weight_bytes(cfg, world, fp8=fp8)
    page = max(1, dense_kv_page_bytes(cfg, world))
    requested = max_pages if max_pages > 0 else batch_size * -(-chunk_size // PAGE_SIZE)
    work = chunk_size * (cfg.hidden_size * 12 + 2 * (cfg.intermediate_size // world) * 4
                         + (cfg.num_attention_heads // world) * cfg.head_dim * 8)
    budget = int(((arena_gb if arena_gb > 0 else device_gb) - reserve_gb) * GIB)
    fit = max(0, (budget - weights - work) // page)
    return MemoryPlan(tp=world, cp=1, ep=False, weights_bytes=weights, page_bytes=page, tokens_per_page=PAGE_SIZE,
                      workspace_bytes=work, budget_bytes=budget, max_pages=int(fit), max_tokens=int(fit) * PAGE_SIZE,
                      requested_pages=requested, requested_fits=requested <= fit)
