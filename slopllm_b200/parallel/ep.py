"""Expert parallelism over NVLink peer memory: dispatch of 4-bit token rows to the ranks that own their experts,
block-scaled grouped GEMMs there, and the weighted combine back at the token's home rank, with no NCCL call and no host
synchronisation (`csrc/ep_dispatch.cu`, `csrc/gemm_fp4_tcgen05.cu`).

A round (one MoE layer) for a rank:

    home tokens --route--> sort by expert --counts--> every rank          (sl_moe_sort_routes, sl_ep_counts_push)
    plan: where my rows start in each owner's sorted receive buffer      (sl_ep_plan, waits for the W count vectors)
    quantise home tokens once, store each routed copy into its owner     (sl_nvfp4_quantize_rows, sl_ep_dispatch)
    wait for all dispatches, gate/up + SiLU * mul, re-quantise, down     (sl_ep_wait, grouped NVFP4 GEMMs)
      ... the down GEMM's epilogue stores every output row into the home rank's combine buffer
    tell the home ranks, wait for mine, weighted sum of my routes        (sl_ep_signal, sl_ep_wait, sl_ep_reduce)

The reference has no expert parallelism (its experts are tensor-parallel, `src/glm51_model.ts:178-232`); the NCCL
all-to-all form of this path is `GlmMoeDsaModel._moe_ep`.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from ..ops import fp4
from ..ops import native as N
from ..ops import tcgen05

MAX_RANKS = 8
vp, i32, u32 = C.c_void_p, C.c_int, C.c_uint32


class EpCtx(C.Structure):
    _fields_ = [("counts", vp * MAX_RANKS), ("flags", vp * MAX_RANKS), ("recv_q", vp * MAX_RANKS), ("recv_sf", vp * MAX_RANKS),
                ("recv_g", vp * MAX_RANKS), ("recv_meta", vp * MAX_RANKS), ("comb", vp * MAX_RANKS), ("epoch", vp), ("done", vp),
                ("status", vp), ("rank", i32), ("world", i32), ("E", i32), ("El", i32), ("cap", i32), ("home_cap", i32), ("K", i32),
                ("H", i32), ("bn", i32), ("max_spins", u32)]


N._SIGS.update({
    "sl_ep_counts_push": [C.POINTER(EpCtx), vp, vp],
    "sl_ep_plan": [C.POINTER(EpCtx), vp, vp, vp, vp, vp],
    "sl_ep_dispatch": [C.POINTER(EpCtx), vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp],
    "sl_ep_wait": [C.POINTER(EpCtx), i32, vp],
    "sl_ep_signal": [C.POINTER(EpCtx), i32, vp],
    "sl_ep_reduce": [C.POINTER(EpCtx), vp, i32, vp, i32, i32, i32, vp],
})


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class EpExchange:
    """Symmetric buffers and the per-round calls of one rank.

    `max_home_tokens`: most tokens this rank is home to in one round; `max_recv_rows`: most routed rows it can receive
    (worst case: every route of the round lands here).  Capacities are fixed, so rounds can be captured in CUDA graphs."""

    def __init__(self, rank: int, world: int, E: int, H: int, top_k: int, max_home_tokens: int, max_recv_rows: int,
                 local: torch.Tensor, peer_ptrs: List[int], bn: int = 128, wait_spins: int = 4_000_000,
                 status: Optional[torch.Tensor] = None):
        assert world <= MAX_RANKS and E % world == 0 and H % 256 == 0
        self.rank, self.world, self.E, self.El, self.H, self.top_k, self.bn = rank, world, E, E // world, H, top_k, bn
        self.cap, self.home_cap = max_recv_rows, max_home_tokens * top_k
        self.local, self.peer_ptrs = local, peer_ptrs
        lay = self.layout(world, E, H, top_k, max_home_tokens, max_recv_rows, bn)
        if local.numel() < lay["total"]:
            raise ValueError(f"symmetric buffer of {local.numel()} bytes is smaller than the EP layout ({lay['total']} bytes)")
        self.lay = lay
        dev = local.device
        self.state = torch.zeros(8, dtype=torch.int32, device=dev)           # [0] epoch, [1] block tickets, [4..7] status
        self.status = status if status is not None else self.state[4:8]
        c = EpCtx(epoch=self.state.data_ptr(), done=self.state.data_ptr() + 4, status=self.status.data_ptr(), rank=rank, world=world,
                  E=E, El=self.El, cap=self.cap, home_cap=self.home_cap, K=H, H=H, bn=bn, max_spins=wait_spins)
        for r in range(world):
            base = peer_ptrs[r]
            for name in ("counts", "flags", "recv_q", "recv_sf", "recv_g", "recv_meta", "comb"):
                getattr(c, name)[r] = base + lay[name]
        self.ctx = c
        self.comb_ptrs = (vp * MAX_RANKS)(*[peer_ptrs[r] + lay["comb"] for r in range(world)] + [0] * (MAX_RANKS - world))

    @staticmethod
    def layout(world, E, H, top_k, max_home_tokens, max_recv_rows, bn) -> dict:
        off = 0
        lay = {}

        def take(name, n):
            nonlocal off
            lay[name] = off
            off += _align(n)
        El = E // world
        take("counts", world * E * 4)
        take("flags", 3 * world * 4)
        take("recv_q", max_recv_rows * (H // 2))
        take("recv_sf", ((max_recv_rows + bn - 1) // bn + El) * (H // 64) * 512)
        take("recv_g", max_recv_rows * 4)
        take("recv_meta", max_recv_rows * 8)
        take("comb", max_home_tokens * top_k * H * 2)
        lay["total"] = off
        return lay

    def _view(self, name: str, nbytes: int, dtype) -> torch.Tensor:
        o = self.lay[name]
        return self.local[o:o + nbytes].view(dtype)

    # ---- the phases of a round (separate so that a test can run W emulated ranks phase by phase) ---------------------
    def route_and_count(self, ids: torch.Tensor):
        """Home side, step 1: sort this rank's routes by global expert and push the per-expert counts to every rank."""
        dev = ids.device
        ids32 = ids.reshape(-1).to(torch.int32).contiguous()
        n = ids32.numel()
        self._n = n
        self._tokens = ids.shape[0]
        scratch = torch.empty(((max(n, 1) + 1023) // 1024) * (self.E + 1), dtype=torch.int32, device=dev)
        self._off_local = torch.zeros(self.E + 1, dtype=torch.int32, device=dev)
        self._order = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
        rows_of = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
        src_tok = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
        if n:
            N.call("sl_moe_sort_routes", ids32.data_ptr(), n, self.top_k, 0, self.E, scratch.data_ptr(), self._off_local.data_ptr(),
                   self._order.data_ptr(), rows_of.data_ptr(), src_tok.data_ptr(), N.stream())
        N.call("sl_ep_counts_push", C.byref(self.ctx), self._off_local.data_ptr(), N.stream())

    def plan_and_dispatch(self, x_home: torch.Tensor):
        """Home side, step 2: wait for every rank's counts, place my rows, quantise my tokens once and store each routed
        copy into its owner's receive buffer."""
        dev = x_home.device
        self._my_off = torch.empty(self.El + 1, dtype=torch.int32, device=dev)
        self._my_pad = torch.empty(self.El + 1, dtype=torch.int32, device=dev)
        dest_row = torch.empty(self.E, dtype=torch.int32, device=dev)
        dest_prow = torch.empty(self.E, dtype=torch.int32, device=dev)
        N.call("sl_ep_plan", C.byref(self.ctx), self._my_off.data_ptr(), self._my_pad.data_ptr(), dest_row.data_ptr(),
               dest_prow.data_ptr(), N.stream())
        T = x_home.shape[0]
        if T:
            q, sf, g = fp4.quantize_rows(x_home, bn=128)
        else:
            q = sf = g = torch.zeros(16, dtype=torch.uint8, device=dev)
        N.call("sl_ep_dispatch", C.byref(self.ctx), q.data_ptr(), sf.data_ptr(), g.data_ptr(), self._order.data_ptr(),
               self._off_local.data_ptr(), dest_row.data_ptr(), dest_prow.data_ptr(), self._n, self.top_k, 128, T, N.stream())

    def experts(self, experts):
        """Owner side: wait for all dispatches, run my experts over the received rows; the down projection's epilogue
        stores into the home ranks' combine buffers; then tell the home ranks."""
        from ..ops.gemm import _sf_tiles_of
        N.call("sl_ep_wait", C.byref(self.ctx), 1, N.stream())
        H, I, cap, bn = self.H, experts.inter, self.cap, self.bn
        dev = self.local.device
        plan = fp4.GroupPlan(self._my_off, self._my_pad, self.El, cap, bn)
        sf13, sf2 = _sf_tiles_of(experts)
        xq = self._view("recv_q", cap * (H // 2), torch.uint8).view(cap, H // 2)
        sfx = self._view("recv_sf", plan.max_row_tiles * (H // 64) * 512, torch.uint8)
        gx = self._view("recv_g", cap * 4, torch.float32)
        act = fp4.grouped_gemm_fp4(experts.w13, sf13, experts.g13, xq, sfx, gx, plan, I, True, fp4.OUT_BF16)
        aq, sfa, ga = fp4.quantize_rows(act, plan=plan, num_rows=self._my_off[self.El:])
        # down projection with the combine epilogue
        max_tiles = plan.max_row_tiles * (H // 128)
        tiles = torch.empty(max_tiles * N.kernels().sl_fp4_tile_bytes(), dtype=torch.uint8, device=dev)
        ntiles = torch.empty(1, dtype=torch.int32, device=dev)
        N.call("sl_fp4_build_tiles", tiles.data_ptr(), ntiles.data_ptr(), plan.offsets.data_ptr(), plan.pad.data_ptr(), plan.groups, H, 0,
               bn, max_tiles, N.stream())
        g2 = experts.g2.to(torch.float32).contiguous()
        N.call("sl_gemm_fp4_tcgen05_scatter", experts.w2.data_ptr(), sf2.data_ptr(), g2.data_ptr(), experts.w2.shape[0] * experts.w2.shape[1],
               aq.data_ptr(), sfa.data_ptr(), ga.data_ptr(), cap, self.peer_ptrs[self.rank] + self.lay["recv_meta"], self.comb_ptrs,
               self.world, H, I, bn, tiles.data_ptr(), ntiles.data_ptr(), max_tiles, tcgen05.error_flag(dev).data_ptr(), N.stream())
        N.call("sl_ep_signal", C.byref(self.ctx), 2, N.stream())

    def combine(self, out_home: torch.Tensor, wts: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
        """Home side, last step: wait for all owners, out_home[t] (+)= sum_j wts[t, j] * (expert output of route (t, j))."""
        N.call("sl_ep_wait", C.byref(self.ctx), 2, N.stream())
        T = out_home.shape[0]
        w = wts.to(torch.float32).contiguous()
        N.call("sl_ep_reduce", C.byref(self.ctx), out_home.data_ptr(), out_home.stride(0), w.data_ptr(), T, self.top_k, int(accumulate),
               N.stream())
        return out_home

    def moe(self, x_home: torch.Tensor, experts, ids: torch.Tensor, wts: torch.Tensor, out_home: torch.Tensor,
            accumulate: bool = False) -> torch.Tensor:
        """All phases in order (one process per rank)."""
        self.route_and_count(ids)
        self.plan_and_dispatch(x_home)
        self.experts(experts)
        return self.combine(out_home, wts, accumulate)

    def check_status(self) -> None:
        st = self.status.tolist()
        if st[0]:
            self.status.zero_()
            raise N.CollectiveTimeout(f"rank {self.rank}: expert-parallel exchange failed at site {st[1]} (expected {st[2]}, saw {st[3]})")


def make_exchange(ctx, cfg, max_tokens: int) -> EpExchange:
    """Allocate and map the symmetric buffers of this job's ranks (`max_tokens`: most tokens of the whole replica in one
    round; every rank is home to ceil(max_tokens / W) of them and may receive all of their routes)."""
    from .nvlink import symmetric_alloc
    W = ctx.world
    home = -(-max_tokens // W)
    recv = max_tokens * cfg.num_experts_per_tok
    lay = EpExchange.layout(W, cfg.n_routed_experts, cfg.hidden_size, cfg.num_experts_per_tok, home, recv, 128)
    buf, ptrs, keep = symmetric_alloc(ctx, lay["total"])
    torch.cuda.synchronize()
    import torch.distributed as dist
    dist.barrier(group=ctx.group)
    ex = EpExchange(ctx.rank, W, cfg.n_routed_experts, cfg.hidden_size, cfg.num_experts_per_tok, home, recv, buf, ptrs, 128,
                    status=tcgen05.error_flag(ctx.device)[12:16])
    ex._keep = keep
    return ex
