"""Process-group plumbing: one process per GPU under `torch.distributed`.

The reference drives N GPUs from one process and infers collectives from tensor tags
(`src/parallel_ops.ts:2362-2470`).  Here every rank is a process (NCCL on GPU, gloo on
CPU); the model calls the collectives it needs explicitly through :class:`Comm`.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from datetime import timedelta
from typing import List, Optional

import torch
import torch.distributed as dist

_PREFILL_AR_FP32 = os.environ.get("SLOPLLM_B200_PREFILL_AR_FP32", "0") == "1"


@dataclass
class ParallelContext:
    rank: int = 0
    world: int = 1
    device: torch.device = torch.device("cpu")
    cp: bool = False           # context parallelism: KV rows interleaved across ranks
    ep: bool = False           # expert parallelism for routed experts
    group: Optional[object] = None
    # data parallelism: the job's ranks are cut into `dp_world` replicas of `world` ranks each; `rank` / `world` / `group`
    # describe this rank's replica, `global_rank` / `global_world` the whole job (None: the replica is the job)
    dp_rank: int = 0
    dp_world: int = 1
    global_rank: Optional[int] = None
    global_world: Optional[int] = None

    def peer(self, i: int) -> int:
        """Job-wide rank of member `i` of this replica (what point-to-point calls and `src=` arguments take)."""
        if self.group is None or self.dp_world == 1:
            return i
        return dist.get_global_rank(self.group, i)

    @property
    def is_distributed(self) -> bool:
        return self.world > 1

    @property
    def cp_world(self) -> int:
        return self.world if self.cp else 1

    @property
    def cp_rank(self) -> int:
        return self.rank if self.cp else 0


def init_from_env(backend: Optional[str] = None, cp: bool = False, ep: bool = False,
                  timeout_s: float = 600.0, dp: int = 1, device_index: Optional[int] = None) -> ParallelContext:
    """Initialise from torchrun's RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* variables.  With `dp` > 1 the ranks form
    `dp` model replicas of WORLD_SIZE / dp consecutive ranks; the returned context is that of this rank's replica.
    `device_index` overrides LOCAL_RANK as this rank's CUDA device (`--gpus 4,5,6,7`)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    use_cuda = torch.cuda.is_available() and backend != "gloo"
    device = torch.device("cuda", local if device_index is None else device_index) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        kw = {"device_id": device} if use_cuda else {}
        dist.init_process_group(backend or ("nccl" if use_cuda else "gloo"), rank=rank, world_size=world,
                                timeout=timedelta(seconds=timeout_s), **kw)
    if dp > 1:
        if world % dp != 0:
            raise ValueError(f"{world} ranks cannot form {dp} replicas of equal size")
        tp = world // dp
        mine = None
        for d in range(dp):                      # every rank creates every group, in the same order
            g = dist.new_group(ranks=list(range(d * tp, (d + 1) * tp)))
            if d == rank // tp:
                mine = g
        return ParallelContext(rank % tp, tp, device, cp, ep, mine if tp > 1 else None, dp_rank=rank // tp, dp_world=dp,
                               global_rank=rank, global_world=world)
    return ParallelContext(rank, world, device, cp, ep, dist.group.WORLD if world > 1 else None)


def shutdown() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()


class Comm:
    """Collectives the model needs, in their unfused (library) form.

    This is the always-correct baseline (NCCL on GPU, gloo on CPU); the fused NVLink
    kernels in :mod:`slopllm_b200.parallel.fused` subclass it and override the hot ones.
    Reference call sites: `src/parallel_ops.ts:219-239` (all-reduce), `:328-420`
    (all-gather), `:2870-3111` (CP merge), `:4233-4330` (top-k owner merge).
    """

    def __init__(self, ctx: ParallelContext):
        self.ctx = ctx

    # -- basic ---------------------------------------------------------------------------
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.ctx.world == 1:
            return x
        y = x.contiguous().clone()
        dist.all_reduce(y, group=self.ctx.group)
        return y

    def all_gather(self, x: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if self.ctx.world == 1:
            return x
        parts = [torch.empty_like(x) for _ in range(self.ctx.world)]
        dist.all_gather(parts, x.contiguous(), group=self.ctx.group)
        return torch.cat(parts, dim=dim)

    def all_gather_list(self, x: torch.Tensor) -> List[torch.Tensor]:
        if self.ctx.world == 1:
            return [x]
        parts = [torch.empty_like(x) for _ in range(self.ctx.world)]
        dist.all_gather(parts, x.contiguous(), group=self.ctx.group)
        return parts

    def all_gather_many(self, xs: List[torch.Tensor], dim: int = -1) -> List[torch.Tensor]:
        """Several tensors gathered by ONE collective: their bytes travel as one packed buffer (segments padded to 16
        bytes) and each result is the concatenation of the ranks' parts along `dim`.  Reference: `allGatherTwo`
        (`src/parallel_ops.ts:2666-2712`, `p2p_allgather_two_write_kernel`), which gathers the two query-side tensors of
        a context-parallel layer in one launch."""
        if self.ctx.world == 1:
            return list(xs)
        segs, sizes = [], []
        for x in xs:
            b = x.contiguous().view(torch.uint8).reshape(-1)
            pad = (-b.numel()) % 16
            segs.append(b if pad == 0 else torch.cat([b, b.new_zeros(pad)]))
            sizes.append((b.numel(), b.numel() + pad))
        parts = self.all_gather_list(torch.cat(segs))
        outs, off = [], 0
        for x, (n, padded) in zip(xs, sizes):
            outs.append(torch.cat([p[off:off + n].view(x.dtype).reshape(x.shape) for p in parts], dim=dim))
            off += padded
        return outs

    def all_to_all(self, send: List[torch.Tensor]) -> List[torch.Tensor]:
        """send[i] goes to rank i; shapes may differ per pair but must be known to both
        sides (callers exchange counts first)."""
        W = self.ctx.world
        if W == 1:
            return send
        if self.ctx.device.type == "cuda":
            # NCCL: exchange the row counts, then one all_to_all_single with per-peer split sizes
            dev = self.ctx.device
            mine = torch.tensor([s.shape[0] for s in send], dtype=torch.int64, device=dev)
            counts = torch.stack(self.all_gather_list(mine)).tolist()            # counts[src][dst]
            in_splits = [int(c) for c in counts[self.ctx.rank]]
            out_splits = [int(counts[peer][self.ctx.rank]) for peer in range(W)]
            tail = tuple(send[0].shape[1:])
            inp = torch.cat([s.contiguous() for s in send], 0) if sum(in_splits) else torch.empty((0,) + tail, dtype=send[0].dtype, device=dev)
            out = torch.empty((sum(out_splits),) + tail, dtype=send[0].dtype, device=dev)
            dist.all_to_all_single(out, inp, out_splits, in_splits, group=self.ctx.group)
            return list(out.split(out_splits, 0))
        recv: List[Optional[torch.Tensor]] = [None] * W
        # gloo has no all_to_all: W broadcast-free rounds of paired send/recv
        counts = self.all_gather_list(torch.tensor([s.shape[0] for s in send], dtype=torch.int64))
        reqs = []
        for peer in range(W):
            n = int(counts[peer][self.ctx.rank])
            recv[peer] = torch.empty((n,) + tuple(send[peer].shape[1:]), dtype=send[peer].dtype)
            if peer == self.ctx.rank:
                recv[peer].copy_(send[peer])
                continue
            reqs.append(dist.isend(send[peer].contiguous(), self.ctx.peer(peer), group=self.ctx.group))
            reqs.append(dist.irecv(recv[peer], self.ctx.peer(peer), group=self.ctx.group))
        for r in reqs:
            r.wait()
        return recv  # type: ignore[return-value]

    def barrier(self) -> None:
        if self.ctx.world > 1:
            dist.barrier(group=self.ctx.group)

    def check_status(self) -> None:
        """Raise if a device-side bounded wait expired (library collectives have none)."""

    def begin_forward(self) -> None:
        """Called at the start of every forward pass (fused communicators rotate buffers)."""

    def partial_sink(self, rows: int, final: bool = False):
        """Where a partial-sum producer should put its result: None = return a tensor."""
        return None

    def cp_merge_partials(self, ops, o_part, lse_part):
        """Merge this rank's split partials across ranks; returns this rank's head slice."""
        o, lse = (ops.combine_f32 if hasattr(ops, "combine_f32") else ops.combine)([o_part], [lse_part])
        return self.cp_merge_heads(ops, o, lse)

    # -- fused-op shaped interface (overridden by the NVLink kernels) -------------------------
    def allreduce_add_rmsnorm(self, ops, partial, residual, weight, eps, want_perm: bool = False):
        """sum over ranks of `partial`, add to `residual`, RMSNorm.  Returns (normed, residual').
        `want_perm`: the consumer is an NVFP4 tensor-core kernel; a CUDA backend then also emits its permuted operand."""
        if want_perm and getattr(ops, "name", "") == "cuda":
            return ops.add_rmsnorm(self._reduce_partial(partial), residual, weight, eps, want_perm=True)
        return ops.add_rmsnorm(self._reduce_partial(partial), residual, weight, eps)

    PREFILL_AR_BF16_MIN_ROWS = 33

    def _reduce_partial(self, partial: torch.Tensor) -> torch.Tensor:
        """Sum of the ranks' partial rows.  Prefill-sized fp32 partials on GPUs cross the links as bf16 (half the bytes of
        the fp32 library all-reduce; the reference's reduce kernels move bf16 too, `csrc/glm_p2p.cu:627-680`); the sum is added
        to the fp32 residual by the norm kernel.  `SLOPLLM_B200_PREFILL_AR_FP32=1` keeps fp32 on the wire."""
        if (self.ctx.world > 1 and partial.is_cuda and partial.dtype == torch.float32
                and partial.shape[0] >= self.PREFILL_AR_BF16_MIN_ROWS and not _PREFILL_AR_FP32):
            y = partial.to(torch.bfloat16)
            dist.all_reduce(y, group=self.ctx.group)
            return y
        return self.all_reduce(partial)

    def cp_merge_heads(self, ops, o: torch.Tensor, lse: torch.Tensor):
        """Merge per-rank attention partials over all heads and return this rank's head
        slice `[T, h/W, R]` (log-sum-exp combine; `csrc/glm_context_parallel.cu:277-540`)."""
        W, r = self.ctx.world, self.ctx.rank
        if W == 1:
            return o
        if o.is_cuda and hasattr(ops, "combine"):
            # every rank needs only its own heads: exchange head slices (all-to-all), then merge the W partials
            T, h, R = o.shape
            hl = h // W
            send_o = o.to(torch.float32).view(T, W, hl, R).permute(1, 0, 2, 3).contiguous()
            send_l = lse.to(torch.float32).view(T, W, hl).permute(1, 0, 2).contiguous()
            recv_o, recv_l = torch.empty_like(send_o), torch.empty_like(send_l)
            dist.all_to_all_single(recv_o, send_o, group=self.ctx.group)
            dist.all_to_all_single(recv_l, send_l, group=self.ctx.group)
            merged, _ = ops.combine([recv_o[i].unsqueeze(2) for i in range(W)], [recv_l[i].unsqueeze(2) for i in range(W)],
                                    want_lse=False)
            return merged
        os_ = torch.stack(self.all_gather_list(o.to(torch.float32)))
        ls_ = torch.stack(self.all_gather_list(lse.to(torch.float32)))
        merged, _ = ops.merge_attention_partials(os_, ls_)
        hl = o.shape[1] // W
        return merged[:, r * hl:(r + 1) * hl].contiguous()

    def cp_merge_topk_all(self, ops, pos: torch.Tensor, score: torch.Tensor, top_k: int) -> torch.Tensor:
        """Global top-k over the ranks' local candidate lists, returned in full on every rank: [T, k] global positions of
        ALL selected keys (-1 padded).  Both the candidates' scores and their positions travel (the gather form of
        context parallelism attends over a replicated copy of the rows, so every rank needs every winner)."""
        W = self.ctx.world
        if W == 1:
            return pos
        T, k = pos.shape
        s = torch.where(pos >= 0, score.to(torch.float32), torch.full_like(score, float("-inf"), dtype=torch.float32))
        alls = torch.cat(self.all_gather_list(s.contiguous()), dim=1)                    # [T, W*k]
        allp = torch.cat(self.all_gather_list(pos.to(torch.int32).contiguous()), dim=1)  # [T, W*k]
        if hasattr(ops, "topk_select_plain") and alls.is_cuda:
            idx = ops.topk_select_plain(alls, top_k).to(torch.int64)                     # ascending candidate index, -1 padded
        else:
            order = torch.sort(alls, dim=1, descending=True, stable=True).indices[:, :top_k]
            idx = torch.sort(order, dim=1).values
        ok = idx >= 0
        out = allp.gather(1, torch.where(ok, idx, torch.zeros_like(idx)))
        # a winner that is a padding candidate (score -inf: fewer than k real candidates overall) carries position -1 already
        return torch.where(ok, out, torch.full_like(out, -1)).to(torch.int32).contiguous()

    def cp_merge_topk(self, ops, pos: torch.Tensor, score: torch.Tensor, top_k: int) -> torch.Tensor:
        """Global top-k over the ranks' local candidate lists (global positions + scores, -1 padded).

        Only the scores travel: every rank gathers all candidate scores [T, W*k], selects the k best of the
        union (the same selection everywhere) and keeps the winners that are its own candidates.  Returns
        [T, k] global positions of THIS rank's selected keys, -1 elsewhere; the caller turns them into local
        cache slots.  Ties go to the lower (rank, candidate index).  Reference: the all-gather + re-select of
        `src/parallel_ops.ts:4233-4330`, which also moves the positions."""
        W, r = self.ctx.world, self.ctx.rank
        if W == 1:
            return pos
        T, k = pos.shape
        s = torch.where(pos >= 0, score.to(torch.float32), torch.full_like(score, float("-inf"), dtype=torch.float32))
        alls = torch.cat(self.all_gather_list(s.contiguous()), dim=1)                   # [T, W*k]
        if hasattr(ops, "topk_select_plain") and alls.is_cuda:
            idx = ops.topk_select_plain(alls, top_k).to(torch.int64)                    # ascending candidate index
        else:
            order = torch.sort(alls, dim=1, descending=True, stable=True).indices[:, :top_k]
            idx = torch.sort(order, dim=1).values
        mine = (idx >= r * k) & (idx < (r + 1) * k)
        local_j = torch.where(mine, idx - r * k, torch.zeros_like(idx))
        out = torch.where(mine, pos.gather(1, local_j).to(torch.int32), torch.full((1,), -1, dtype=torch.int32, device=pos.device))
        return out.contiguous()
