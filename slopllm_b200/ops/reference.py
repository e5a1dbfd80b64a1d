"""Plain PyTorch fp32 reference of every op.

This module is (1) the op set the CPU backend runs (gloo plumbing model, scheduler tests)
and (2) the oracle each CUDA kernel is compared against.  All functions accept CPU or
CUDA tensors, compute in fp32 and return fp32 unless noted.  Shapes use
T = tokens in the step, H = hidden, h = heads, R = kv_lora_rank, Dr = rope dim.

Math follows the reference model (`src/glm51_model.ts:577-942`) and its kernels
(`csrc/glm_ops.cu`, `csrc/glm_indexer.cu`, `csrc/glm_sampling.cu`).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import quant

# ---- normalisation ---------------------------------------------------------------------


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.to(torch.float32)
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return xf * inv * weight.to(torch.float32)


def add_rmsnorm(x: torch.Tensor, residual: Optional[torch.Tensor], weight: torch.Tensor, eps: float):
    """residual' = residual + x ; out = rmsnorm(residual').  Returns (out, residual')."""
    r = x.to(torch.float32) if residual is None else residual.to(torch.float32) + x.to(torch.float32)
    return rmsnorm(r, weight, eps), r


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.to(torch.float32)
    mu = xf.mean(-1, keepdim=True)
    var = (xf - mu).pow(2).mean(-1, keepdim=True)
    return (xf - mu) * torch.rsqrt(var + eps) * weight.to(torch.float32) + bias.to(torch.float32)


def rmsnorm_gated(x, gate, weight, eps):
    """norm(x) * w * silu(gate)  (Gated DeltaNet output norm, `csrc/glm_gdn.cu:495`)."""
    return rmsnorm(x, weight, eps) * torch.nn.functional.silu(gate.to(torch.float32))


# ---- rotary embedding ---------------------------------------------------------------------


def rope_cos_sin(positions: torch.Tensor, rope_dim: int, theta: float):
    inv_freq = 1.0 / (theta ** (torch.arange(0, rope_dim, 2, dtype=torch.float32, device=positions.device) / rope_dim))
    ang = positions.to(torch.float32).unsqueeze(-1) * inv_freq
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, positions: torch.Tensor, theta: float, rope_dim: int, interleave: bool) -> torch.Tensor:
    """Rotate the first `rope_dim` values of the last dim.  x: [T, ..., D].

    `interleave=True` pairs (2i, 2i+1) (GLM `rope_interleave`); otherwise pairs
    (i, i + rope_dim/2)  (reference `csrc/glm_ops.cu:1876`).
    """
    xf = x.to(torch.float32)
    cos, sin = rope_cos_sin(positions, rope_dim, theta)           # [T, rope_dim/2]
    while cos.dim() < xf.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    rot, rest = xf[..., :rope_dim], xf[..., rope_dim:]
    if interleave:
        a, b = rot[..., 0::2], rot[..., 1::2]
        out = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2)
    else:
        half = rope_dim // 2
        a, b = rot[..., :half], rot[..., half:]
        out = torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)
    return torch.cat([out, rest], dim=-1)


# ---- linear ----------------------------------------------------------------------------------


def linear(x: torch.Tensor, w) -> torch.Tensor:
    """y = x @ W^T for a :class:`LinearWeight` or a plain `[N, K]` tensor."""
    wf = w.dequant(torch.float32) if hasattr(w, "dequant") else w.to(torch.float32)
    return x.to(torch.float32) @ wf.t()


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    g, u = gate_up.to(torch.float32).chunk(2, dim=-1)
    return torch.nn.functional.silu(g) * u


# ---- MoE routing --------------------------------------------------------------------------------


def moe_route(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, n_group: int = 1,
              topk_group: int = 1, norm_topk: bool = True, scale: float = 1.0):
    """Sigmoid routing with bias-corrected, group-limited top-k.

    scores = sigmoid(logits); choice by scores + bias (restricted to the `topk_group`
    best groups, a group's rank being the sum of its top-2 biased scores); weights = the
    unbiased scores of the chosen, normalised to 1, times `scale`.  Ties pick the lower
    expert id.  Reference: `src/tensor.ts:688`, `csrc/glm_ops.cu:2343-2416`.
    Returns (ids int32 [T, k], weights f32 [T, k]).
    """
    s = torch.sigmoid(logits.to(torch.float32))
    choice = s if bias is None else s + bias.to(torch.float32)
    T, E = s.shape
    if n_group > 1:
        g = choice.reshape(T, n_group, E // n_group)
        gscore = g.topk(min(2, E // n_group), dim=-1).values.sum(-1)
        gsel = _stable_topk(gscore, topk_group)
        gmask = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, gsel, True)
        choice = torch.where(gmask.unsqueeze(-1).expand_as(g), g, torch.full_like(g, float("-inf"))).reshape(T, E)
    ids = _stable_topk(choice, top_k)
    w = s.gather(1, ids)
    if norm_topk:
        w = w / w.sum(-1, keepdim=True).clamp(min=1e-20)
    return ids.to(torch.int32), w * scale


def _stable_topk(x: torch.Tensor, k: int) -> torch.Tensor:
    """Top-k indices, descending by value, ties broken towards the lower index."""
    order = torch.sort(x, dim=-1, descending=True, stable=True).indices
    return order[..., :k]


def moe_experts(x: torch.Tensor, experts, ids: torch.Tensor, weights: torch.Tensor,
                col_slice: Optional[Tuple[int, int]] = None, a4: bool = False) -> torch.Tensor:
    """Σ_k w_k · down_e(silu(gate_e x) · up_e x) over the routed experts of each token.

    `experts` is an :class:`ExpertWeights` (possibly TP-sliced on the intermediate dim, in
    which case the result is this rank's partial sum).  `a4` emulates the W4A4 path of the block-scaled tensor-core
    kernels: the token rows and the intermediate activations go through NVFP4 (as bf16 rows) before each product.
    """
    xf = x.to(torch.float32)
    if a4:
        xf = quant.nvfp4_fake_quant_rows(x.to(torch.bfloat16))
    out = torch.zeros(x.shape[0], experts.hidden, dtype=torch.float32, device=x.device)
    for e in torch.unique(ids).tolist():
        tok, slot = (ids == e).nonzero(as_tuple=True)
        w13, w2 = experts.dequant_expert(int(e))
        h = silu_mul(xf[tok] @ w13.t())
        if a4:
            h = quant.nvfp4_fake_quant_rows(h.to(torch.bfloat16))
        y = h @ w2.t()
        if a4:
            y = y.to(torch.bfloat16).to(torch.float32)
        out.index_add_(0, tok, y * weights[tok, slot].unsqueeze(-1))
    return out


# ---- paged KV helpers ------------------------------------------------------------------------------


def token_slots(page_table: torch.Tensor, batch_idx: torch.Tensor, positions: torch.Tensor,
                page_size: int, cp_world: int = 1, cp_rank: int = 0):
    """Physical slot (page*page_size + offset) of each token's KV row on this rank.

    Under context parallelism token p lives on rank ``p % W`` at local position ``p // W``
    (reference `csrc/glm_flash.cu:1150-1170`).  Returns (slots int64 [T], owned bool [T]).
    """
    pos = positions.to(torch.int64)
    owned = (pos % cp_world) == cp_rank
    local = pos // cp_world
    page = page_table.to(torch.int64)[batch_idx.to(torch.int64), local // page_size]
    return page * page_size + local % page_size, owned


def kv_append(cache: torch.Tensor, rows: torch.Tensor, slots: torch.Tensor, owned: torch.Tensor) -> None:
    """cache: u8 [num_slots, row_bytes]; write the owned rows."""
    cache[slots[owned]] = rows[owned]


# ---- DSA indexer ---------------------------------------------------------------------------------------


def indexer_quantize_q(q: torch.Tensor, head_weights: torch.Tensor, head_dim_scale: float):
    """Quantise indexer queries `[T, Hi, D]` to e4m3 with one power-of-two scale per
    (token, head) and fold that scale and `head_dim_scale` into the per-head weights.

    Returns (q8 as f32 values [T, Hi, D], effective weights f32 [T, Hi]).
    Reference: `csrc/glm_indexer.cu:1338-1374`.
    """
    q8, scale = quant.fp8_quantize_block(q.to(torch.bfloat16), q.shape[-1], pow2=True)
    return q8.to(torch.float32), head_weights.to(torch.float32) * scale.squeeze(-1) * head_dim_scale


def indexer_scores(q8: torch.Tensor, w_eff: torch.Tensor, k_rows: torch.Tensor, dim: int) -> torch.Tensor:
    """score[t, j] = Σ_h w_eff[t,h] · relu(q8[t,h]·k8[j]) · kscale[j] for packed key rows
    `[J, D+4]`.  Returns f32 [T, J]."""
    k8 = k_rows[..., :dim].contiguous().view(torch.float8_e4m3fn).to(torch.float32)
    ks = k_rows[..., dim:dim + 4].contiguous().view(torch.float32).squeeze(-1)
    dots = torch.einsum("thd,jd->thj", q8, k8)
    return (torch.relu(dots) * w_eff.unsqueeze(-1)).sum(1) * ks.unsqueeze(0)


def select_topk_ascending(scores: torch.Tensor, valid: torch.Tensor, k: int) -> torch.Tensor:
    """Per row: indices of the `min(k, #valid)` best valid scores, ascending by index,
    padded with -1.  Ties prefer the lower index.  Returns int32 [T, k]."""
    T, J = scores.shape
    s = torch.where(valid, scores, torch.full_like(scores, float("-inf")))
    kk = min(k, J)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :kk]
    ok = valid.gather(1, order)
    idx = torch.where(ok, order, torch.full_like(order, J + 1))
    idx = torch.sort(idx, dim=-1).values
    idx = torch.where(idx > J, torch.full_like(idx, -1), idx)
    if kk < k:
        idx = torch.cat([idx, torch.full((T, k - kk), -1, dtype=idx.dtype, device=idx.device)], 1)
    return idx.to(torch.int32)


def indexer_topk(q8, w_eff, index_cache, page_table, batch_idx, positions, top_k: int, page_size: int,
                 dim: int, cp_world: int = 1, cp_rank: int = 0):
    """Causal top-k over this rank's key shard.

    Returns (global token positions int32 [T, top_k] ascending, -1 padded; their scores f32
    [T, top_k]).  A query that sees at most `top_k` keys in total (position + 1 <= top_k)
    selects every visible key without scoring (scores 0) - the CUDA kernel does the same.
    Causal limits are in global coordinates: local key j is global position j*W + rank
    (reference `csrc/glm_indexer.cu` `idx_local_causal_limit`).
    """
    T = q8.shape[0]
    out = torch.full((T, top_k), -1, dtype=torch.int32, device=q8.device)
    out_s = torch.zeros((T, top_k), dtype=torch.float32, device=q8.device)
    for t in range(T):
        b, p = int(batch_idx[t]), int(positions[t])
        n_local = (p - cp_rank) // cp_world + 1 if p >= cp_rank else 0
        if n_local <= 0:
            continue
        j = torch.arange(n_local, device=q8.device)
        if p + 1 <= top_k:
            sel = j
        else:
            slots = page_table[b].to(torch.int64)[j // page_size] * page_size + j % page_size
            sc = indexer_scores(q8[t:t + 1], w_eff[t:t + 1], index_cache[slots], dim)
            sel = select_topk_ascending(sc, torch.ones_like(sc, dtype=torch.bool), top_k)[0].to(torch.int64)
            sel = sel[sel >= 0]
            out_s[t, : sel.numel()] = sc[0, sel]
        out[t, : sel.numel()] = (sel * cp_world + cp_rank).to(torch.int32)
    return out, out_s


def topk_to_slots(topk_pos: torch.Tensor, page_table: torch.Tensor, batch_idx: torch.Tensor,
                  page_size: int, cp_world: int = 1):
    """Global positions -> local physical slots, with ordered compaction of -1 entries.

    Returns (slots int32 [T, k] (-1 padded), lengths int32 [T]).
    Reference: `csrc/glm_indexer.cu:303-376`.
    """
    T, k = topk_pos.shape
    valid = topk_pos >= 0
    local = torch.div(topk_pos.clamp(min=0).to(torch.int64), cp_world, rounding_mode="floor")
    pt = page_table.to(torch.int64)[batch_idx.to(torch.int64)]          # [T, P]
    page = pt.gather(1, (local // page_size).clamp(max=pt.shape[1] - 1))
    slots = torch.where(valid, page * page_size + local % page_size, torch.full_like(local, -1))
    # stable compaction: valid entries first, original order kept
    order = torch.sort((~valid).to(torch.int8), dim=1, stable=True).indices
    return slots.gather(1, order).to(torch.int32), valid.sum(1).to(torch.int32)


# ---- attention ---------------------------------------------------------------------------------------------


def sparse_mla(q_abs: torch.Tensor, q_pe: torch.Tensor, kv_cache: torch.Tensor, slots: torch.Tensor,
               lengths: torch.Tensor, sm_scale: float, kv_lora: int, rope_dim: int, group: int = 128):
    """Sparse MLA over gathered packed rows.

    q_abs [T, h, R], q_pe [T, h, Dr], kv_cache u8 [num_slots, row_bytes], slots int32 [T, k].
    Returns (o f32 [T, h, R], lse f32 [T, h]) with lse = log Σ exp (natural log); rows with
    no key give o = 0, lse = -inf.
    """
    T, h, R = q_abs.shape
    o = torch.zeros(T, h, R, dtype=torch.float32, device=q_abs.device)
    lse = torch.full((T, h), float("-inf"), dtype=torch.float32, device=q_abs.device)
    qa, qp = q_abs.to(torch.float32), q_pe.to(torch.float32)
    for t in range(T):
        n = int(lengths[t])
        if n == 0:
            continue
        rows = kv_cache[slots[t, :n].to(torch.int64)]
        ckv, kpe = quant.unpack_kv_rows(rows, kv_lora, rope_dim, group)
        s = (qa[t] @ ckv.t() + qp[t] @ kpe.t()) * sm_scale           # [h, n]
        lse[t] = torch.logsumexp(s, dim=-1)
        o[t] = torch.softmax(s, dim=-1) @ ckv
    return o, lse


def merge_attention_partials(o_parts: torch.Tensor, lse_parts: torch.Tensor):
    """Log-sum-exp merge of W partial results.  o_parts [W, T, h, R], lse_parts [W, T, h].
    Reference: `csrc/glm_context_parallel.cu:39-160`."""
    m = lse_parts.max(0).values
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp(lse_parts - m_safe)                                 # exp(-inf) = 0
    denom = w.sum(0)
    o = (o_parts.to(torch.float32) * w.unsqueeze(-1)).sum(0) / denom.clamp(min=1e-38).unsqueeze(-1)
    lse = torch.where(denom > 0, m_safe + torch.log(denom.clamp(min=1e-38)), torch.full_like(m, float("-inf")))
    return o, lse


def v_expand(o: torch.Tensor, w_v: torch.Tensor) -> torch.Tensor:
    """out[t, h, :] = o[t, h, :R] @ w_v[h]  with w_v [h, R, Dv].  Returns [T, h*Dv]."""
    return torch.einsum("thr,hrv->thv", o.to(torch.float32), w_v.to(torch.float32)).flatten(1)


def absorb_q(q_nope: torch.Tensor, w_kn: torch.Tensor) -> torch.Tensor:
    """q_abs[t, h] = q_nope[t, h, :Dn] @ w_kn[h] with w_kn [h, Dn, R]."""
    return torch.einsum("thd,hdr->thr", q_nope.to(torch.float32), w_kn.to(torch.float32))


def dense_attention(q, k, v, sm_scale, causal_offset: int = 0):
    """Plain causal attention for the dense families.  q [Tq, h, D], k/v [Tk, hk, D]."""
    Tq, h, D = q.shape
    Tk, hk, _ = k.shape
    rep = h // hk
    kf = k.to(torch.float32).repeat_interleave(rep, dim=1)
    vf = v.to(torch.float32).repeat_interleave(rep, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.to(torch.float32), kf) * sm_scale
    qi = torch.arange(Tq, device=q.device).unsqueeze(1) + causal_offset
    ki = torch.arange(Tk, device=q.device).unsqueeze(0)
    s = s.masked_fill(ki > qi, float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vf)


# ---- sampling -------------------------------------------------------------------------------------------------


def lowbias32(x: torch.Tensor) -> torch.Tensor:
    """32-bit integer hash used as the counter RNG (`csrc/glm_sampling.cu:54-70`)."""
    x = x.to(torch.int64) & 0xFFFFFFFF
    x = ((x ^ (x >> 16)) * 0x7FEB352D) & 0xFFFFFFFF
    x = ((x ^ (x >> 15)) * 0x846CA68B) & 0xFFFFFFFF
    return x ^ (x >> 16)


def uniform_from_counter(counter: int, rows: torch.Tensor, stream: int = 0) -> torch.Tensor:
    """Uniform (0,1) per row from (counter, row, stream)."""
    h = lowbias32(lowbias32(rows.to(torch.int64) * 0x9E3779B1 + counter) + stream * 0x85EBCA6B)
    return (h.to(torch.float64) + 0.5) / 4294967296.0


def apply_penalties(logits: torch.Tensor, history: torch.Tensor, hist_len: torch.Tensor,
                    rep: torch.Tensor, presence: torch.Tensor) -> torch.Tensor:
    """Repetition (divide positive / multiply negative) and presence (subtract) penalties
    over each row's recent-token window.  history int [B, Wd] (-1 = empty)."""
    out = logits.to(torch.float32).clone()
    B, V = out.shape
    for b in range(B):
        n = int(hist_len[b])
        if n == 0:
            continue
        toks = torch.unique(history[b, :n][history[b, :n] >= 0]).to(torch.int64)
        v = out[b, toks]
        r = float(rep[b])
        v = torch.where(v > 0, v / r, v * r) - float(presence[b])
        out[b, toks] = v
    return out


def sample_distribution(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                        max_k: int = 64):
    """Candidate set after temperature → top-k (≤ max_k) → top-p.

    Returns (ids int64 [B, max_k], probs f32 [B, max_k]) sorted by descending probability,
    zero probability outside the kept set.  Rows with temperature 0 keep only the argmax.
    """
    B, V = logits.shape
    lf = logits.to(torch.float32)
    kk = min(max_k, V)
    vals, ids = torch.sort(lf, dim=-1, descending=True, stable=True)
    vals, ids = vals[:, :kk], ids[:, :kk]
    t = temperature.to(torch.float32).clamp(min=1e-6).unsqueeze(-1)
    k_eff = torch.where(top_k <= 0, torch.full_like(top_k, kk), top_k.clamp(max=kk)).unsqueeze(-1)
    greedy = (temperature <= 0).unsqueeze(-1)
    k_eff = torch.where(greedy, torch.ones_like(k_eff), k_eff)
    rank = torch.arange(kk, device=logits.device).unsqueeze(0)
    keep = rank < k_eff
    p = torch.softmax(torch.where(keep, vals / t, torch.full_like(vals, float("-inf"))), dim=-1)
    csum = p.cumsum(-1)
    # keep the smallest prefix whose mass reaches top_p (always at least one candidate)
    keep_p = (csum - p) < top_p.to(torch.float32).unsqueeze(-1)
    p = torch.where(keep & keep_p, p, torch.zeros_like(p))
    p = p / p.sum(-1, keepdim=True)
    return ids, p


def sample_from_candidates(ids: torch.Tensor, probs: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """Inverse-CDF draw per row with uniforms u [B]."""
    csum = probs.to(torch.float64).cumsum(-1)
    pick = (csum < u.to(torch.float64).unsqueeze(-1) * csum[:, -1:]).sum(-1).clamp(max=ids.shape[1] - 1)
    # never pick a zero-probability candidate
    pick = torch.minimum(pick, (probs > 0).sum(-1) - 1).clamp(min=0)
    return ids.gather(1, pick.unsqueeze(-1)).squeeze(-1)


def spec_reject_linear(draft_tokens, draft_ids, draft_probs, target_ids, target_probs, u_accept, u_resample):
    """Linear-chain speculative rejection sampling (`csrc/glm_sampling.cu:644-706`).

    draft_tokens [B, D]; draft_ids/probs [B, D, C] the draft candidate sets the tokens were
    drawn from; target_ids/probs [B, D+1, C] the target candidate sets at each position;
    u_accept [B, D], u_resample [B, D+1] uniforms.
    For i < D: accept draft token x with prob min(1, p_t(x)/p_d(x)); on the first
    rejection sample from norm(max(p_t - p_d, 0)) and stop; if all are accepted sample the
    bonus token from the target distribution at position D.
    Returns (out_tokens int64 [B, D+1] (-1 padded), num_accepted int64 [B]).
    """
    B, D = draft_tokens.shape
    out = torch.full((B, D + 1), -1, dtype=torch.int64)
    nacc = torch.zeros(B, dtype=torch.int64)
    for b in range(B):
        i = 0
        while i < D:
            x = int(draft_tokens[b, i])
            pt = float(target_probs[b, i][target_ids[b, i] == x].sum())
            pd = float(draft_probs[b, i][draft_ids[b, i] == x].sum())
            if pd > 0 and float(u_accept[b, i]) < min(1.0, pt / pd):
                out[b, i] = x
                i += 1
                continue
            # residual distribution over the target candidate set
            tid, tp = target_ids[b, i], target_probs[b, i].to(torch.float64)
            dp = torch.zeros_like(tp)
            for c in range(tid.numel()):
                m = draft_ids[b, i] == tid[c]
                if m.any():
                    dp[c] = draft_probs[b, i][m].sum()
            res = (tp - dp).clamp(min=0)
            if float(res.sum()) <= 0:
                res = tp
            out[b, i] = int(sample_from_candidates(tid.unsqueeze(0), res.unsqueeze(0).to(torch.float32),
                                                   u_resample[b, i:i + 1])[0])
            break
        else:
            out[b, D] = int(sample_from_candidates(target_ids[b, D].unsqueeze(0), target_probs[b, D].unsqueeze(0),
                                                   u_resample[b, D:D + 1])[0])
        nacc[b] = i
    return out, nacc


# ---- recurrent families (Qwen3.5 Gated DeltaNet, glm5_next KDA / mHC) ----------------------------------------------


def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], state: Optional[torch.Tensor] = None,
                  activation: bool = True):
    """Depthwise causal conv over time.  x [T, C], weight [C, Kw], state [C, Kw-1] (previous
    inputs).  Returns (y [T, C], new_state).  Reference `csrc/glm_gdn.cu:359-494`."""
    T, C = x.shape
    Kw = weight.shape[1]
    xf = x.to(torch.float32)
    st = torch.zeros(C, Kw - 1, dtype=torch.float32, device=x.device) if state is None else state.to(torch.float32)
    full = torch.cat([st.t(), xf], dim=0)                            # [Kw-1+T, C]
    win = full.unfold(0, Kw, 1)                                      # [T, C, Kw]
    y = (win * weight.to(torch.float32).unsqueeze(0)).sum(-1)
    if bias is not None:
        y = y + bias.to(torch.float32)
    if activation:
        y = torch.nn.functional.silu(y)
    return y, full[-(Kw - 1):].t().contiguous()


def gdn_recurrent(q, k, v, g, beta, state):
    """Gated DeltaNet recurrence, one token at a time.

    q,k [T, h, Dk] (L2-normalised by the caller), v [T, h, Dv], g [T, h] (log decay ≤ 0),
    beta [T, h], state [h, Dk, Dv].  S ← exp(g)·S ; S ← S + k ⊗ β(v − Sᵀk) ; o = Sᵀ q.
    Reference `csrc/glm_gdn.cu:68-207` (step) and `:208` (prefill scan).
    """
    T, h, Dk = q.shape
    S = state.to(torch.float32).clone()
    out = torch.empty(T, h, v.shape[-1], dtype=torch.float32, device=q.device)
    qf, kf, vf = q.to(torch.float32), k.to(torch.float32), v.to(torch.float32)
    for t in range(T):
        S = S * torch.exp(g[t].to(torch.float32)).view(h, 1, 1)
        kv = torch.einsum("hk,hkv->hv", kf[t], S)
        delta = (vf[t] - kv) * beta[t].to(torch.float32).unsqueeze(-1)
        S = S + torch.einsum("hk,hv->hkv", kf[t], delta)
        out[t] = torch.einsum("hk,hkv->hv", qf[t], S)
    return out, S


def kda_scan(q, k, v, forget, beta, A_log, dt_bias, state, lower_bound: float):
    """KDA recurrence (`csrc/glm_flash_hybrid.cu:31-72`): q, k L2-normalised (eps 1e-6 inside the
    root), q scaled by Dk^-0.5; per-channel decay exp(lower_bound * sigmoid(exp(A_log[h]) *
    (forget + dt_bias[h, :]))) with lower_bound < 0; beta = bf16(sigmoid(beta logits)).
    q, k, forget [T, h, Dk], v [T, h, Dv], beta [T, h], dt_bias [h, Dk], state [h, Dk, Dv]."""
    T, h, Dk = q.shape
    S = state.to(torch.float32).clone()
    out = torch.empty(T, h, v.shape[-1], dtype=torch.float32, device=q.device)
    qf, kf, vf = q.to(torch.float32), k.to(torch.float32), v.to(torch.float32)
    qf = qf / torch.sqrt((qf * qf).sum(-1, keepdim=True) + 1e-6) * Dk ** -0.5
    kf = kf / torch.sqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)
    decay = torch.exp(lower_bound * torch.sigmoid(torch.exp(A_log.to(torch.float32)).view(1, h, 1)
                                                   * (forget.to(torch.float32) + dt_bias.to(torch.float32).view(1, h, Dk))))
    bt = torch.sigmoid(beta.to(torch.float32)).to(torch.bfloat16).to(torch.float32)
    for t in range(T):
        S = S * decay[t].unsqueeze(-1)
        kv = torch.einsum("hk,hkv->hv", kf[t], S)
        delta = (vf[t] - kv) * bt[t].unsqueeze(-1)
        S = S + torch.einsum("hk,hv->hkv", kf[t], delta)
        out[t] = torch.einsum("hk,hkv->hv", qf[t], S)
    return out, S


def kda_norm(x, gate, weight, eps):
    """Sigmoid-gated RMSNorm (`csrc/glm_flash_hybrid.cu:73-83`)."""
    return rmsnorm(x, weight, eps) * torch.sigmoid(gate.to(torch.float32))


def mhc_pre(x: torch.Tensor, fn: torch.Tensor, base: torch.Tensor, scale: torch.Tensor, norm_eps: float, hc_eps: float,
            iters: int):
    """Manifold hyper-connection, pre-sublayer (`csrc/glm_flash_hybrid.cu:84-142`).

    x [T, 4, H] residual streams, fn [24, 4H] coefficient projection, base [24], scale [3].
    Returns (collapsed [T, H], post [T, 4], comb [T, 4, 4]): the sublayer input, the weights
    that add the sublayer output back to each stream and the stream-mixing matrix
    (softmax rows + eps, then alternating column / row normalisation)."""
    T, n, H = x.shape
    xf = x.to(torch.float32).reshape(T, n * H)
    inv = torch.rsqrt((xf * xf).mean(-1, keepdim=True) + norm_eps)
    logits = (xf * inv) @ fn.to(torch.float32).t()                            # [T, 24]
    base, scale = base.to(torch.float32), scale.to(torch.float32)
    pre = torch.sigmoid(logits[:, :4] * scale[0] + base[:4]) + hc_eps
    post = 2.0 * torch.sigmoid(logits[:, 4:8] * scale[1] + base[4:8])
    mix = torch.softmax((logits[:, 8:24] * scale[2] + base[8:24]).view(T, 4, 4), -1) + hc_eps
    for it in range(iters):
        if it > 0:
            mix = mix / (mix.sum(-1, keepdim=True) + hc_eps)
        mix = mix / (mix.sum(-2, keepdim=True) + hc_eps)
    collapsed = torch.einsum("ts,tsh->th", pre, x.to(torch.float32))
    return collapsed, post, mix


def mhc_post(residual: torch.Tensor, block: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    """out[t, s] = post[t, s] * block[t] + sum_i comb[t, i, s] * residual[t, i]  (`:143-154`)."""
    return post.unsqueeze(-1) * block.to(torch.float32).unsqueeze(1) + torch.einsum("tis,tih->tsh", comb, residual.to(torch.float32))


def mhc_streams(x: torch.Tensor, expand: bool) -> torch.Tensor:
    """expand: [T, H] -> 4 identical streams [T, 4, H]; collapse: mean of the streams (`:155-170`)."""
    if expand:
        return x.unsqueeze(1).expand(-1, 4, -1).contiguous()
    return x.to(torch.float32).mean(1)


def log_softmax_nll(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    return -torch.log_softmax(logits.to(torch.float32), -1).gather(1, targets.unsqueeze(-1).to(torch.int64)).squeeze(-1)


def next_pow2(n: int) -> int:
    return 1 << max(0, (int(n) - 1).bit_length())


def padded_kv_len(n: int) -> int:
    """Graph-variant bucket for KV length (`src/execution-workspace.ts:162-165`)."""
    return max(1024, next_pow2(n))


_ = math
