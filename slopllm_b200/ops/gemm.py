"""Large-M (prefill) linear layers and grouped expert GEMMs on the tcgen05 tensor cores.

Dense bf16 weights go straight through `sl_gemm_bf16_tcgen05` (TMA-fed, TMEM accumulators).
NVFP4 weights go through `sl_gemm_w4_tcgen05` / `sl_grouped_gemm_w4_tcgen05`, which expand the
packed weight tile to f16 on its way into shared memory (W4A16, the reference's numerics:
`csrc/glm_mma_moe_coop.cu:351` also turns FP4 into a 16-bit type before its MMA); shapes those
kernels do not take (K not a multiple of 64) fall back to `sl_nvfp4_dequant_bf16` + the bf16 GEMM.
The MoE layer runs as two *grouped* GEMMs over the expert-sorted token rows with a device-built
tile table (reference: sort + `grouped_mma_kernel` + unscatter, `csrc/glm_mma_moe.cu:110-619`).
`SLOPLLM_B200_W4_GEMM=0` forces the expansion path (comparison runs).
"""
from __future__ import annotations

import torch

import os

from . import native as N
from . import tcgen05

DEQUANT_BUDGET_BYTES = 3 << 30          # transient bf16 copy of expert weights per grouped launch
W4_GEMM = os.environ.get("SLOPLLM_B200_W4_GEMM", "1") != "0"
W4_DENSE_MAX_ROWS = 256                 # plain (non-grouped) NVFP4 linears take the fused kernel up to this many rows
# prefill MoE on the block-scaled FP4 tensor cores: activations are quantised to NVFP4 on the fly (W4A4).
# SLOPLLM_B200_MOE_A4=0 keeps 16-bit activations (W4A16, the reference's numerics) on the expansion kernels.
MOE_A4 = os.environ.get("SLOPLLM_B200_MOE_A4", "1") != "0"
OUT_BF16, OUT_F32, OUT_F16 = 0, 1, 2


def _w4_ok(K: int) -> bool:
    return W4_GEMM and K % 64 == 0


def to_f16_rows(x: torch.Tensor, src_rows: torch.Tensor | None = None, rows: int | None = None) -> torch.Tensor:
    """f16 copy of bf16 rows, optionally gathered: out[m] = x[src_rows[m]] (rows outside x give zeros)."""
    M = x.shape[0] if src_rows is None else (src_rows.numel() if rows is None else rows)
    H = x.shape[1]
    out = torch.empty(M, H, dtype=torch.float16, device=x.device)
    N.call("sl_gather_rows_f16", out.data_ptr(), x.data_ptr(), N.ptr(src_rows), M, H, x.stride(0), x.shape[0], N.stream())
    return out


def _out_tensor(M: int, Nn: int, out_kind: int, dev) -> torch.Tensor:
    dt = {OUT_BF16: torch.bfloat16, OUT_F32: torch.float32, OUT_F16: torch.float16}[out_kind]
    pad = 4 if out_kind == OUT_F32 else 8
    ld = (Nn + pad - 1) // pad * pad
    return torch.empty(M, ld, dtype=dt, device=dev)[:, :Nn]


def gemm_w4(x16: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor, gs: torch.Tensor, out_kind: int, split: int = 0) -> torch.Tensor:
    """y = x16 @ dequant(W)^T with W = NVFP4 [Nn, K/2] + e4m3 [Nn, K/16]; gs holds 1 global scale, or 2 with `split`
    (output columns below `split` use the first)."""
    M, K = x16.shape
    Nn = wq.shape[0]
    gs = gs.to(torch.float32).reshape(-1).contiguous()
    y = _out_tensor(M, Nn, out_kind, x16.device)
    bn = 256 if Nn >= 512 else 128
    N.call("sl_gemm_w4_tcgen05", x16.data_ptr(), wq.data_ptr(), ws.data_ptr(), gs.data_ptr(), gs.numel(), split, y.data_ptr(),
           M, Nn, K, x16.stride(0), y.stride(0), out_kind, tcgen05.error_flag(x16.device).data_ptr(), bn, N.stream())
    return y


def grouped_gemm_w4(a16: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor, gs: torch.Tensor, offsets: torch.Tensor, out_kind: int,
                    split: int = 0, bn: int = 0) -> torch.Tensor:
    """Grouped form of `gemm_w4`: rows [offsets[g], offsets[g+1]) of a16 use weight matrix g of the stacks
    wq [G, Nn, K/2], ws [G, Nn, K/16], gs [G] or [G, 2]."""
    M, K = a16.shape
    G, Nn, _ = wq.shape
    gs = gs.to(torch.float32).contiguous()
    g_per = gs.numel() // G
    c = _out_tensor(M, Nn, out_kind, a16.device)
    if bn == 0:
        bn = 256 if Nn >= 512 else 128
    ncol = (Nn + bn - 1) // bn
    max_tiles = ((M + 127) // 128 + G) * ncol
    tiles = torch.empty(max_tiles, 4, dtype=torch.int32, device=a16.device)
    ntiles = torch.empty(1, dtype=torch.int32, device=a16.device)
    N.call("sl_build_group_tiles", tiles.data_ptr(), ntiles.data_ptr(), offsets.data_ptr(), G, Nn, max_tiles, bn, N.stream())
    N.call("sl_grouped_gemm_w4_tcgen05", a16.data_ptr(), wq.data_ptr(), ws.data_ptr(), gs.data_ptr(), g_per, split, c.data_ptr(),
           M, Nn, K, a16.stride(0), c.stride(0), out_kind, tiles.data_ptr(), ntiles.data_ptr(), max_tiles,
           tcgen05.error_flag(a16.device).data_ptr(), bn, N.stream())
    return c


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
    # One weight matrix shared by many rows: expanding it once (a few MB) and running the bf16 GEMM at 1.0 - 1.2 PFLOP/s beats
    # the in-kernel expansion, whose converter warps cap it near 0.45 PFLOP/s; the fused kernel wins when a matrix meets few rows.
    if (w.is_nvfp4 and x.shape[0] <= W4_DENSE_MAX_ROWS and _w4_ok(x.shape[1]) and x.dtype == torch.bfloat16
            and x.stride(0) % 8 == 0):
        return gemm_w4(to_f16_rows(x), w.weight, w.scale, w.scale2, OUT_F32 if out_f32 else OUT_BF16)
    return tcgen05.gemm_bf16(x, _weight_bf16(w), out_f32)


def grouped_gemm(a: torch.Tensor, b_stack: torch.Tensor, offsets: torch.Tensor, out_f32: bool, bn: int = 0) -> torch.Tensor:
    """C[r] = A[r] @ B[g(r)]^T where rows [offsets[g], offsets[g+1]) belong to group g.
    a [M, K] bf16, b_stack [G, Nn, K] bf16, offsets int32 [G + 1] on the device."""
    M, K = a.shape
    G, Nn, _ = b_stack.shape
    c = torch.empty(M, Nn, dtype=torch.float32 if out_f32 else torch.bfloat16, device=a.device)
    # 128 x 256 tiles measured faster than 128 x 128 for both expert GEMMs of a prefill chunk
    if bn == 0:
        bn = 256 if Nn >= 512 else 128
    ncol = (Nn + bn - 1) // bn
    max_tiles = ((M + 127) // 128 + G) * ncol
    tiles = torch.empty(max_tiles, 4, dtype=torch.int32, device=a.device)
    ntiles = torch.empty(1, dtype=torch.int32, device=a.device)
    N.call("sl_build_group_tiles", tiles.data_ptr(), ntiles.data_ptr(), offsets.data_ptr(), G, Nn, max_tiles, bn, N.stream())
    N.call("sl_grouped_gemm_bf16_tcgen05", a.data_ptr(), b_stack.data_ptr(), c.data_ptr(), M, Nn, K, a.stride(0), K, c.stride(0),
           int(out_f32), G, tiles.data_ptr(), ntiles.data_ptr(), max_tiles, tcgen05.error_flag(a.device).data_ptr(), bn, N.stream())
    return c


def _sf_tiles_of(experts):
    """Scale tiles of an expert stack for the block-scaled kernel, made once and kept with the weights."""
    from . import fp4
    t = getattr(experts, "_sf_tiles", None)
    if t is None:
        t = (fp4.sf_tiles(experts.s13), fp4.sf_tiles(experts.s2))
        experts._sf_tiles = t
    return t


def fp4_moe_ok(experts, H: int) -> bool:
    from . import fp4
    I = experts.inter
    return bool(MOE_A4 and experts.is_nvfp4 and fp4.shapes_ok(I, H) and fp4.shapes_ok(H, I) and I % 128 == 0)


def experts_fp4(experts, xq3, plan, out_kind: int = OUT_BF16) -> torch.Tensor:
    """SwiGLU experts over expert-sorted, NVFP4-quantised rows `xq3` = (codes, scale tiles, global scales) laid out for
    `plan`: gate/up with the SiLU * mul epilogue, re-quantisation of the activations, down projection.
    Returns [rows, H] (bf16 or fp32)."""
    from . import fp4
    sf13, sf2 = _sf_tiles_of(experts)
    xq, sfx, gx = xq3
    act = fp4.grouped_gemm_fp4(experts.w13, sf13, experts.g13, xq, sfx, gx, plan, experts.inter, True, fp4.OUT_BF16)
    aq, sfa, ga = fp4.quantize_rows(act, plan=plan)
    return fp4.grouped_gemm_fp4(experts.w2, sf2, experts.g2, aq, sfa, ga, plan, experts.hidden, False, out_kind)


def moe_large(ops, x, experts, shared, ids, wts) -> torch.Tensor:
    """Expert MLP for many tokens: routes sorted by expert on the device, gate/up and down as grouped GEMMs over
    the sorted rows (NVFP4 experts: weights expanded inside the GEMM; otherwise bf16 weights, expanded in groups
    that bound the transient copy), SiLU·mul in between, weighted un-sort into the shared expert's result.
    Returns fp32 [T, H] (this rank's partial sum)."""
    T, H = x.shape
    k = ids.shape[1]
    E, I = experts.num_experts, experts.inter
    dev = x.device
    xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
    # stable counting sort of the routes by expert on the device: offsets [E + 1], sorted row -> token, route -> sorted row
    ids32 = ids.reshape(-1).to(torch.int32).contiguous()
    M = ids32.numel()
    scratch = torch.empty(((M + 1023) // 1024) * (E + 1), dtype=torch.int32, device=dev)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    order = torch.empty(M, dtype=torch.int32, device=dev)
    rows_of = torch.empty(M, dtype=torch.int32, device=dev)
    src_tok = torch.empty(M, dtype=torch.int32, device=dev)
    N.call("sl_moe_sort_routes", ids32.data_ptr(), M, k, experts.expert_offset, E, scratch.data_ptr(), offsets.data_ptr(),
           order.data_ptr(), rows_of.data_ptr(), src_tok.data_ptr(), N.stream())
    wts = wts.to(torch.float32).contiguous()
    use_fp4 = fp4_moe_ok(experts, H) and xb.stride(-1) == 1
    # the shared expert writes the fp32 result first, the routed experts accumulate into it
    out = _shared_expert_large(xb, shared, use_fp4) if shared is not None else None
    if out is not None and (out.stride(0) != H or out.dtype != torch.float32):
        out = out.to(torch.float32).contiguous()
    acc = 0 if out is None else 1
    if out is None:
        out = torch.empty(T, H, dtype=torch.float32, device=dev)
    if use_fp4:
        # tokens gathered into expert order and quantised in one pass; both expert GEMMs on tcgen05 kind::mxf4nvf4
        # every token row is quantised once; the experts get copies of the 4-bit rows in expert order
        from . import fp4
        plan = fp4.group_plan(offsets, E, M)
        xq_tok = getattr(xb, "_sl_fp4", None) or fp4.quantize_rows(xb, bn=128)
        xb._sl_fp4 = None
        y = experts_fp4(experts, fp4.gather_rows(*xq_tok, 128, src_tok, plan), plan)
        N.call("sl_moe_unsort_reduce", out.data_ptr(), y.data_ptr(), rows_of.data_ptr(), wts.data_ptr(), T, k, H, acc, 1, N.stream())
        return out
    if experts.is_nvfp4 and _w4_ok(H) and _w4_ok(I) and xb.stride(0) % 8 == 0:
        # weights expanded inside the GEMMs: no transient bf16 copy, activations in f16
        xs16 = to_f16_rows(xb, src_tok)                                           # [T*k, H] expert-sorted rows
        h = grouped_gemm_w4(xs16, experts.w13, experts.s13, experts.g13, offsets, OUT_F16, split=I)
        act16 = torch.empty(M, I, dtype=torch.float16, device=dev)
        N.call("sl_silu_mul_h", act16.data_ptr(), h.data_ptr(), M, I, N.stream())
        y = grouped_gemm_w4(act16, experts.w2, experts.s2, experts.g2, offsets, OUT_BF16)
        N.call("sl_moe_unsort_reduce", out.data_ptr(), y.data_ptr(), rows_of.data_ptr(), wts.data_ptr(), T, k, H, acc, 1, N.stream())
        return out
    xs = xb.index_select(0, src_tok)                                              # [T*k, H] expert-sorted rows
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
    N.call("sl_moe_unsort_reduce", out.data_ptr(), y.data_ptr(), rows_of.data_ptr(), wts.data_ptr(), T, k, H, acc, 1, N.stream())
    return out


def _shared_expert_large(xb: torch.Tensor, shared, use_fp4: bool = False) -> torch.Tensor:
    """Shared expert over all rows (one weight matrix, many rows: the block-scaled FP4 path, or expansion + bf16 GEMM).
    Returns fp32 [T, H]."""
    T = xb.shape[0]
    if use_fp4 and fp4_moe_ok(shared, xb.shape[1]):
        from . import fp4
        xq_tok = fp4.quantize_rows(xb, bn=128)
        xb._sl_fp4 = xq_tok                              # the routed experts of the same layer reuse it
        return experts_fp4(shared, xq_tok, fp4.single_group(T, xb.device, 128), OUT_F32)
    if shared.is_nvfp4:
        w13 = dequant_bf16(shared.w13[0], shared.s13[0], shared.g13[0], g_per=2, split=shared.inter)
        w2 = dequant_bf16(shared.w2[0], shared.s2[0], shared.g2[0].reshape(1))
    else:
        w13, w2 = shared.w13[0], shared.w2[0]
    h = tcgen05.gemm_bf16(xb, w13, False)
    hs = torch.empty(T, shared.inter, dtype=torch.bfloat16, device=xb.device)
    if h.stride(0) != h.shape[1]:
        h = h.contiguous()
    N.call("sl_silu_mul", hs.data_ptr(), h.data_ptr(), T, shared.inter, N.stream())
    return tcgen05.gemm_bf16(hs, w2, True)
