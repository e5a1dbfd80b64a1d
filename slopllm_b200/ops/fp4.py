"""NVFP4 x NVFP4 products on the block-scaled tensor-core path (`csrc/gemm_fp4_tcgen05.cu`): weights stay packed E2M1
with their UE4M3 block scales, activation rows are quantised to the same format on the fly (W4A4), and
`tcgen05.mma.kind::mxf4nvf4` applies both sets of scales inside the instruction.

The reference keeps activations in 16 bits and expands the weights before its MMA (`csrc/glm_mma_moe_coop.cu:351`);
this path trades a small, bounded activation error for tensor-core rates that the expansion cannot reach.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import native as N
from . import tcgen05

vp, i32 = N.vp, N.i32
N._SIGS.update({
    "sl_fp4_group_pad": [vp, vp, i32, i32, vp],
    "sl_fp4_build_tiles": [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp],
    "sl_gemm_fp4_tcgen05": [vp, vp, vp, i32, vp, vp, vp, i32, vp, i32, i32, i32, i32, i32, vp, vp, i32, vp, vp],
    "sl_nvfp4_sf_tiles": [vp, vp, i32, i32, i32, vp],
    "sl_nvfp4_gather_rows": [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, vp, i32, i32, vp],
    "sl_nvfp4_quantize_rows": [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, i32, i32, vp, vp],
    "sl_gemm_fp4_tcgen05_scatter": [vp, vp, vp, i32, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, vp, vp, i32, vp, vp],
    "sl_fp4_decode_plan": [vp, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, i32, vp],
    "sl_gemm_fp4_tcgen05_tab": [vp, vp, vp, i32, vp, vp, vp, i32, vp, vp, vp, i32, vp, i32, i32, vp, i32, i32, i32, vp, vp, i32, vp, vp],
})

OUT_BF16, OUT_F32 = 0, 1


def shapes_ok(rows: int, K: int) -> bool:
    """Weight matrices the block-scaled kernel takes: whole 128-row tiles, reduction length a multiple of 256."""
    return rows % 128 == 0 and K % 256 == 0 and K > 0


def sf_tiles(scale: torch.Tensor) -> torch.Tensor:
    """Row-major e4m3 block scales [..., rows, K/16] -> the 512-byte tile layout the kernel loads (one uint8 tensor)."""
    s8 = scale.contiguous().view(torch.uint8)
    *lead, rows, kb = s8.shape
    mats = 1
    for d in lead:
        mats *= d
    out = torch.empty(mats * rows * kb, dtype=torch.uint8, device=s8.device)
    N.call("sl_nvfp4_sf_tiles", out.data_ptr(), s8.data_ptr(), mats, rows, kb * 16, N.stream())
    return out


def pick_bn(rows_per_group: float) -> int:
    return 128 if rows_per_group > 64 else (64 if rows_per_group > 32 else 32)


@dataclass
class GroupPlan:
    """Token rows [offsets[g], offsets[g+1]) belong to group g; `pad[g]` is the group's first row once every group is
    rounded up to a multiple of `bn` rows (the coordinate the activation scale tiles are stored in)."""

    offsets: torch.Tensor          # int32 [G + 1], device
    pad: torch.Tensor              # int32 [G + 1], device
    groups: int
    rows: int
    bn: int

    @property
    def max_row_tiles(self) -> int:
        return (self.rows + self.bn - 1) // self.bn + self.groups


def group_plan(offsets: torch.Tensor, groups: int, rows: int, bn: int = 0) -> GroupPlan:
    bn = bn or pick_bn(rows / max(1, groups))
    pad = torch.empty(groups + 1, dtype=torch.int32, device=offsets.device)
    N.call("sl_fp4_group_pad", pad.data_ptr(), offsets.data_ptr(), groups, bn, N.stream())
    return GroupPlan(offsets, pad, groups, rows, bn)


_single = {}


def single_group(rows: int, device, bn: int = 0) -> GroupPlan:
    """Plan of one group that holds all rows (plain products); kept per shape, so repeated calls upload nothing."""
    bn = bn or pick_bn(rows)
    key = (rows, bn, str(device))
    plan = _single.get(key)
    if plan is None:
        padded = (rows + bn - 1) // bn * bn
        plan = GroupPlan(torch.tensor([0, rows], dtype=torch.int32, device=device),
                         torch.tensor([0, padded], dtype=torch.int32, device=device), 1, rows, bn)
        if len(_single) < 256:
            _single[key] = plan
    return plan


def quantize_rows(x: torch.Tensor, src: Optional[torch.Tensor] = None, rows: Optional[int] = None, terms: int = 1,
                  plan: Optional[GroupPlan] = None, bn: int = 128,
                  num_rows: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """bf16 rows -> (codes u8 [M * terms, K/2], scale tiles u8, global scales f32 [M * terms]).
    With `src` output row m quantises x[src[m]] (a gather, e.g. into expert-sorted order); with `terms` > 1 rows
    m + j * M hold the j-th residual of row m, so that the sum of the terms approaches the 16-bit value.  The scale tiles
    are laid out for GEMM tiles of `bn` token rows: of `plan` (grouped rows), or of one group starting at row 0."""
    assert x.dtype == torch.bfloat16 and x.stride(-1) == 1
    M = x.shape[0] if src is None else (src.numel() if rows is None else rows)
    K = x.shape[1]
    dev = x.device
    if plan is not None:
        assert terms == 1 and plan.rows == M
        bn, row_tiles = plan.bn, plan.max_row_tiles
    else:
        row_tiles = (M * terms + bn - 1) // bn
    q = torch.empty(M * terms, K // 2, dtype=torch.uint8, device=dev)
    # grouped rows leave padding rows between groups and residual terms share tiles: those scale tiles start zeroed; plain
    # rows need no clearing (the kernel zeroes the last tile's padding rows; tiles past `num_rows` are never read)
    sf = (torch.zeros if plan is not None or terms > 1 or bn == 64 else torch.empty)(row_tiles * (K // 64) * 512, dtype=torch.uint8, device=dev)
    g = torch.empty(M * terms, dtype=torch.float32, device=dev)
    N.call("sl_nvfp4_quantize_rows", q.data_ptr(), sf.data_ptr(), g.data_ptr(), x.data_ptr(), N.ptr(src), M, x.shape[0], K,
           x.stride(0), terms, N.ptr(plan.offsets) if plan else 0, N.ptr(plan.pad) if plan else 0, plan.groups if plan else 1, bn,
           N.ptr(num_rows), N.stream())
    return q, sf, g


def gather_rows(q: torch.Tensor, sf: torch.Tensor, g: torch.Tensor, src_bn: int, src: torch.Tensor, plan: GroupPlan):
    """Rows already quantised (ungrouped, scale tiles for `src_bn`-row tiles) gathered into the grouped order of `plan`:
    row m of the result is source row src[m].  Quantising each token once and copying its 4-bit row to every expert it was
    routed to moves a quarter of the bytes that quantising the gathered 16-bit rows would."""
    M, K = src.numel(), q.shape[1] * 2
    dev = q.device
    qo = torch.empty(M, K // 2, dtype=torch.uint8, device=dev)
    sfo = torch.zeros(plan.max_row_tiles * (K // 64) * 512, dtype=torch.uint8, device=dev)
    go = torch.empty(M, dtype=torch.float32, device=dev)
    N.call("sl_nvfp4_gather_rows", qo.data_ptr(), sfo.data_ptr(), go.data_ptr(), q.data_ptr(), sf.data_ptr(), g.data_ptr(),
           src.data_ptr(), M, q.shape[0], K, src_bn, plan.offsets.data_ptr(), plan.pad.data_ptr(), plan.groups, plan.bn, N.stream())
    return qo, sfo, go


def scales_row_major(sf: torch.Tensor, rows: int, K: int, bn: int) -> torch.Tensor:
    """Scale tiles of ungrouped rows (as `quantize_rows` without a plan writes them) -> row-major e4m3 bytes [rows, K/16]."""
    kt = K // 64
    t = sf.view(-1, kt, 32, 4, 4)                       # [tile, k-step, r % 32, r / 32, scale]
    r = torch.arange(rows, device=sf.device)
    tile, rr = r // bn, r % bn
    return t[tile, :, rr % 32, rr // 32, :].reshape(rows, kt * 4).contiguous()


def grouped_gemm_fp4(wq: torch.Tensor, sfa: torch.Tensor, gA: torch.Tensor, xq: torch.Tensor, sfb: torch.Tensor, gB: torch.Tensor,
                     plan: GroupPlan, Nn: int, pair: bool, out_kind: int = OUT_BF16) -> torch.Tensor:
    """out[r, :Nn] for token rows r in [offsets[g], offsets[g+1]) = X[r] . W[g]^T (pair: silu(gate) * up).
    wq [G, Nn (pair: 2 Nn), K/2] packed weights, sfa their scale tiles (`sf_tiles`), gA [G] (pair: [G, 2]) fp32;
    xq / sfb / gB from `quantize_rows` with the same plan."""
    K = wq.shape[-1] * 2
    M = xq.shape[0]
    dev = xq.device
    bn = plan.bn
    pad = 4 if out_kind == OUT_F32 else 8
    ld = (Nn + pad - 1) // pad * pad
    out = torch.empty(M, ld, dtype=torch.float32 if out_kind == OUT_F32 else torch.bfloat16, device=dev)[:, :Nn]
    max_tiles = plan.max_row_tiles * (Nn // 128)
    tile_bytes = N.kernels().sl_fp4_tile_bytes()
    tiles = torch.empty(max_tiles * tile_bytes, dtype=torch.uint8, device=dev)
    ntiles = torch.empty(1, dtype=torch.int32, device=dev)
    N.call("sl_fp4_build_tiles", tiles.data_ptr(), ntiles.data_ptr(), plan.offsets.data_ptr(), plan.pad.data_ptr(), plan.groups, Nn,
           int(pair), bn, max_tiles, N.stream())
    gA = gA.to(torch.float32).contiguous()
    w_rows = wq.shape[0] * wq.shape[1]
    N.call("sl_gemm_fp4_tcgen05", wq.data_ptr(), sfa.data_ptr(), gA.data_ptr(), w_rows, xq.data_ptr(), sfb.data_ptr(), gB.data_ptr(),
           M, out.data_ptr(), out.stride(0), out_kind, K, Nn if pair else 0, bn, tiles.data_ptr(), ntiles.data_ptr(), max_tiles,
           tcgen05.error_flag(dev).data_ptr(), N.stream())
    return out


def gemm_fp4(wq: torch.Tensor, sfa: torch.Tensor, gA: torch.Tensor, xq: torch.Tensor, sfb: torch.Tensor, gB: torch.Tensor,
             out_kind: int = OUT_BF16, bn: int = 128) -> torch.Tensor:
    """Plain product: one weight matrix wq [Nn, K/2], all token rows (quantised with the same `bn`, no plan)."""
    plan = single_group(xq.shape[0], xq.device, bn)
    return grouped_gemm_fp4(wq.unsqueeze(0), sfa, gA.reshape(1), xq, sfb, gB, plan, wq.shape[0], False, out_kind)
