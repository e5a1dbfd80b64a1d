"""Large-M (prefill) linear layers and grouped expert GEMMs on the tcgen05 tensor cores.

Dense bf16 weights go straight through `sl_gemm_bf16_tcgen05` (TMA-fed, TMEM accumulators).
NVFP4 weights are first expanded to bf16 by `sl_nvfp4_dequant_bf16` (W4A16, the reference's
numerics: `csrc/glm_mma_moe_coop.cu:351` also turns FP4 into BF16 before its MMA) and the MoE
layer runs as two *grouped* GEMMs over the expert-sorted token rows with a device-built tile
table (reference: sort + `grouped_mma_kernel` + unscatter, `csrc/glm_mma_moe.cu:110-619`).
"""
from __future__ import annotations

import torch

from . import native as N
from . import tcgen05

DEQUANT_BUDGET_BYTES = 3 << 30          # transient bf16 copy of expert weights per grouped launch


def dequant_bf16(wp: torch.Tensor, scale: torch.Tensor, g: torch.Tensor, g_per: int = 1, split: int = 0) -> torch.Tensor:
    """NVFP4 [..., N, K/2] (+ e4m3 [..., N, K/16], f32 global scales) -> bf16 [..., N, K]."""
    *lead, n, kh = wp.shape
    mats = 1
    for d in lead:
        mats *= d
    K = kh * 2
    out = torch.empty(*lead, n, K, dtype=torch.bfloat16, device=wp.device)
    g = g.to(torch.float32).contiguous()
    N.call("sl_nvfp4_dequant_bf16", out.data_ptr(), wp.data_ptr(), scale.data_ptr(), g.data_ptr(), mats, n, K, g_per, split,
           N.stream())
    return out


def _weight_bf16(w) -> torch.Tensor:
    if w.is_nvfp4:
        return dequant_bf16(w.weight, w.scale, w.scale2.reshape(1))
    return w.weight


def gemm_large(x: torch.Tensor, w, out_f32: bool = False) -> torch.Tensor:
    """y = x @ W^T for T > 32 rows."""
    return tcgen05.gemm_bf16(x, _weight_bf16(w), out_f32)


def grouped_gemm(a: torch.Tensor, b_stack: torch.Tensor, offsets: torch.Tensor, out_f32: bool, bn: int = 0) -> torch.Tensor:
    """C[r] = A[r] @ B[g(r)]^T where rows [offsets[g], offsets[g+1]) belong to group g.
    a [M, K] bf16, b_stack [G, Nn, K] bf16, offsets int32 [G + 1] on the device."""
    M, K = a.shape
    G, Nn, _ = b_stack.shape
    c = torch.empty(M, Nn, dtype=torch.float32 if out_f32 else torch.bfloat16, device=a.device)
    # short reductions are dominated by the per-tile set-up and the output store: use 128 x 256 tiles there
    if bn == 0:
        bn = 256 if (K <= 1024 and Nn >= 1024) else 128
    ncol = (Nn + bn - 1) // bn
    max_tiles = ((M + 127) // 128 + G) * ncol
    tiles = torch.empty(max_tiles, 4, dtype=torch.int32, device=a.device)
    ntiles = torch.empty(1, dtype=torch.int32, device=a.device)
    N.call("sl_build_group_tiles", tiles.data_ptr(), ntiles.data_ptr(), offsets.data_ptr(), G, Nn, max_tiles, bn, N.stream())
    N.call("sl_grouped_gemm_bf16_tcgen05", a.data_ptr(), b_stack.data_ptr(), c.data_ptr(), M, Nn, K, a.stride(0), K, c.stride(0),
           int(out_f32), G, tiles.data_ptr(), ntiles.data_ptr(), max_tiles, tcgen05.error_flag(a.device).data_ptr(), bn, N.stream())
    return c


def moe_large(ops, x, experts, shared, ids, wts) -> torch.Tensor:
    """Expert MLP for many tokens: routes sorted by expert, gate/up and down as grouped GEMMs over
    the sorted rows (experts in groups that bound the transient bf16 weight copy), SiLU·mul in
    between, weighted un-sort at the end.  Returns fp32 [T, H] (this rank's partial sum)."""
    T, H = x.shape
    k = ids.shape[1]
    E, I = experts.num_experts, experts.inter
    dev = x.device
    xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
    flat = ids.reshape(-1).to(torch.int64) - experts.expert_offset
    mine = (flat >= 0) & (flat < E)
    key = torch.where(mine, flat, torch.full_like(flat, E))
    order = torch.argsort(key, stable=True)
    counts = torch.bincount(key, minlength=E + 1)[:E]
    offsets = torch.zeros(E + 1, dtype=torch.int32, device=dev)
    offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device=dev)
    rows_of = torch.where(mine, inv, torch.full_like(inv, -1)).to(torch.int32).contiguous()
    xs = xb.index_select(0, torch.div(order, k, rounding_mode="floor"))          # [T*k, H] expert-sorted rows
    M = xs.shape[0]
    per_expert = 3 * I * H * 2
    group = max(1, min(E, DEQUANT_BUDGET_BYTES // max(1, per_expert)))
    y = torch.empty(M, H, dtype=torch.bfloat16, device=dev)     # per-route outputs; the weighted un-sort accumulates in fp32
    act = torch.empty(M, I, dtype=torch.bfloat16, device=dev)
    for g0 in range(0, E, group):
        g1 = min(E, g0 + group)
        off = offsets[g0:g1 + 1].contiguous()
        if experts.is_nvfp4:
            w13 = dequant_bf16(experts.w13[g0:g1], experts.s13[g0:g1], experts.g13[g0:g1], g_per=2, split=I)
            w2 = dequant_bf16(experts.w2[g0:g1], experts.s2[g0:g1], experts.g2[g0:g1])
        else:
            w13, w2 = experts.w13[g0:g1], experts.w2[g0:g1]
        h = grouped_gemm(xs, w13, off, False)                                      # rows of other groups are left untouched
        N.call("sl_silu_mul", act.data_ptr(), h.data_ptr(), M, I, N.stream())
        yg = grouped_gemm(act, w2, off, False)
        if group >= E:
            y = yg
        else:                                                                      # keep only this group's rows
            lo, hi = int(offsets[g0]), int(offsets[g1])
            y[lo:hi] = yg[lo:hi]
    out = torch.empty(T, H, dtype=torch.float32, device=dev)
    wts = wts.to(torch.float32).contiguous()
    N.call("sl_moe_unsort_reduce", out.data_ptr(), y.data_ptr(), rows_of.data_ptr(), wts.data_ptr(), T, k, H, 0, 1, N.stream())
    if shared is not None:
        if shared.is_nvfp4:
            w13 = dequant_bf16(shared.w13[0], shared.s13[0], shared.g13[0], g_per=2, split=shared.inter)
            w2 = dequant_bf16(shared.w2[0], shared.s2[0], shared.g2[0].reshape(1))
        else:
            w13, w2 = shared.w13[0], shared.w2[0]
        h = tcgen05.gemm_bf16(xb, w13, False)
        hs = torch.empty(T, shared.inter, dtype=torch.bfloat16, device=dev)
        if h.stride(0) != h.shape[1]:
            h = h.contiguous()
        N.call("sl_silu_mul", hs.data_ptr(), h.data_ptr(), T, shared.inter, N.stream())
        out += tcgen05.gemm_bf16(hs, w2, True)
    return out
