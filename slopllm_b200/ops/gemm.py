"""Large-M (prefill) linear layers and grouped expert GEMMs.

Dense bf16 and NVFP4 weights go through the tcgen05 GEMM kernels in `csrc/gemm_tcgen05.cu`
(TMA-fed, TMEM accumulators).  NVFP4 weights are expanded to bf16 tiles on the way into
shared memory (W4A16), matching the reference's numerics (`csrc/glm_mma_moe_coop.cu:351`
dequantises FP4 to BF16 before its `mma.sync`).
"""
from __future__ import annotations

import torch

from . import native as N
from . import quant


def _dequant_bf16(w) -> torch.Tensor:
    if w.is_nvfp4:
        return quant.nvfp4_dequantize(w.weight, w.scale, w.scale2, torch.bfloat16)
    return w.weight


def gemm_large(x: torch.Tensor, w, out_f32: bool = False) -> torch.Tensor:
    """y = x @ W^T for T > 32 rows."""
    from . import tcgen05
    wb = _dequant_bf16(w)
    return tcgen05.gemm_bf16(x, wb, out_f32)


def moe_large(ops, x, experts, shared, ids, wts) -> torch.Tensor:
    """Grouped expert MLP for many tokens: rows are sorted by expert, each expert's block
    runs gate/up -> SiLU·mul -> down on the tensor cores, outputs are scattered back with
    the routing weights.  Returns fp32 [T, H]."""
    from . import tcgen05
    T, H = x.shape
    k = ids.shape[1]
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    lo, hi = experts.expert_offset, experts.expert_offset + experts.num_experts
    flat = ids.reshape(-1).to(torch.int64)
    mine = (flat >= lo) & (flat < hi)
    order = torch.argsort(torch.where(mine, flat, torch.full_like(flat, hi)), stable=True)
    counts = torch.bincount((flat[mine] - lo), minlength=experts.num_experts).tolist()
    tok = torch.div(order, k, rounding_mode="floor")
    wflat = wts.reshape(-1)[order]
    xb = x.to(torch.bfloat16)
    start = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        rows = tok[start:start + n]
        w13, w2 = _expert_bf16(experts, e)
        h = tcgen05.gemm_bf16(xb[rows], w13, False)
        I = h.shape[1] // 2
        act = torch.empty(n, I, dtype=torch.bfloat16, device=x.device)
        N.call("sl_silu_mul", act.data_ptr(), h.data_ptr(), n, I, N.stream())
        y = tcgen05.gemm_bf16(act, w2, True)
        out.index_add_(0, rows, y * wflat[start:start + n].unsqueeze(-1))
        start += n
    if shared is not None:
        w13, w2 = _expert_bf16(shared, 0)
        h = tcgen05.gemm_bf16(xb, w13, False)
        I = h.shape[1] // 2
        act = torch.empty(T, I, dtype=torch.bfloat16, device=x.device)
        N.call("sl_silu_mul", act.data_ptr(), h.data_ptr(), T, I, N.stream())
        out += tcgen05.gemm_bf16(act, w2, True)
    return out


def _expert_bf16(experts, e: int):
    if not experts.is_nvfp4:
        return experts.w13[e], experts.w2[e]
    I = experts.inter
    g = experts.g13[e].to(torch.float32)
    w13 = quant.nvfp4_dequantize(experts.w13[e], experts.s13[e], 1.0)
    w13 = torch.cat([w13[:I] * g[0], w13[I:] * g[1]]).to(torch.bfloat16)
    w2 = quant.nvfp4_dequantize(experts.w2[e], experts.s2[e], experts.g2[e], torch.bfloat16)
    return w13, w2
