"""In-kernel NVLink / NVSwitch collectives over symmetric peer memory.

Every rank allocates the same symmetric buffer (`torch.distributed._symmetric_memory`: CUDA VMM
allocations whose handles are exchanged over the process group, every peer mapped into every
rank's address space).  Kernels then move data themselves:

* fused all-reduce + residual add + RMSNorm: the *producing* kernel (NVFP4 / bf16 linear, MoE
  down-projection) stores its fp32 partial rows directly into each rank's receive slot and
  publishes an epoch flag; the *consuming* kernel waits for the flags (bounded), sums the
  slots in rank order, adds the residual and normalises.  No NCCL call, no separate copy.
* context-parallel attention merge and all-gathers by peer stores (`sl_cp_merge_push`,
  `sl_gather_push`).

Three receive buffers rotate A, B, A, B, ..., C within one forward pass (C = the final norm),
so a rank can never overwrite a slot that a slower peer is still reading: between two uses of
the same buffer every rank has passed a wait that needs all peers' later flags.

Prefill-sized partial sums (more than `MAX_ROWS` rows) take the bulk path when `SLOPLLM_B200_BULK_AR=1`: the tcgen05 GEMM's
epilogue stores its bf16 tile rows into the staging area of the rank that owns them (reduce-scatter inside the GEMM,
tile by tile), the owner sums and stores the result on every rank (all-gather), and the residual add + RMSNorm kernel
waits for the rows it needs (`BulkSink`, `csrc/bulk_collective.cu`).  It is off by default: the default is NCCL.

Plain peer loads/stores only (no multimem, no TMA multicast).  `Comm` (NCCL) stays available as
the fallback and A/B baseline (`fused=False`).  Reference: `csrc/glm_p2p.cu`,
`src/parallel_ops.ts:246-324, 2912-2975`.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import native as N
from .dist import Comm, ParallelContext

MAX_RANKS = 8
vp, i32, u32 = C.c_void_p, C.c_int, C.c_uint32


class PushCtx(C.Structure):
    _fields_ = [("bufs", vp * MAX_RANKS), ("flags", vp * MAX_RANKS), ("epoch", vp), ("block_counter", vp),
                ("rank", i32), ("world", i32), ("slot_rows", i32), ("row_len", i32)]


class RecvCtx(C.Structure):
    _fields_ = [("buf", vp), ("flags", vp), ("epoch", vp), ("done_counter", vp), ("status", vp), ("world", i32),
                ("slot_rows", i32), ("row_len", i32), ("max_spins", u32)]


class CpPushCtx(C.Structure):
    _fields_ = [("o_stage", vp * MAX_RANKS), ("lse_stage", vp * MAX_RANKS), ("flags", vp * MAX_RANKS), ("epoch", vp),
                ("block_counter", vp), ("rank", i32), ("world", i32), ("Tmax", i32), ("h", i32), ("hl", i32), ("R", i32)]


class GatherPushCtx(C.Structure):
    _fields_ = [("bufs", vp * MAX_RANKS), ("flags", vp * MAX_RANKS), ("epoch", vp), ("block_counter", vp), ("rank", i32),
                ("world", i32), ("slot_bytes", C.c_size_t)]


class BulkCtx(C.Structure):
    _fields_ = [("stage", vp * MAX_RANKS), ("rs_count", vp * MAX_RANKS), ("full", vp * MAX_RANKS), ("ag_count", vp * MAX_RANKS),
                ("rs_done", vp), ("ag_done", vp), ("status", vp), ("rank", i32), ("world", i32), ("slot_rows", i32),
                ("row_len", i32), ("max_spins", u32)]


N._SIGS.update({
    "sl_gemm_bf16_tcgen05_rs": [vp, vp, i32, i32, i32, i32, i32, vp, i32, C.POINTER(PushCtx), vp],
    "sl_rs_push_rows": [C.POINTER(BulkCtx), vp, i32, i32, vp],
    "sl_rs_reduce_ag": [C.POINTER(BulkCtx), vp],
    "sl_bulk_add_rmsnorm": [C.POINTER(BulkCtx), vp, vp, vp, vp, C.c_float, vp],
    "sl_ar_add_rmsnorm": [C.POINTER(RecvCtx), vp, vp, vp, vp, i32, i32, C.c_float, vp, vp],
    "sl_push_rows": [C.POINTER(PushCtx), vp, i32, i32, vp],
    "sl_flag_barrier": [C.POINTER(vp), vp, i32, i32, u32, u32, vp, vp],
    "sl_wait_flag": [vp, u32, u32, vp, vp],
    "sl_cp_merge_push": [C.POINTER(CpPushCtx), vp, vp, i32, vp],
    "sl_epoch_wait": [vp, vp, i32, u32, vp, i32, vp],
    "sl_gather_push": [C.POINTER(GatherPushCtx), vp, C.c_size_t, vp],
    "sl_linear_nvfp4_mma_push": [vp, vp, vp, vp, vp, i32, i32, i32, i32, C.POINTER(PushCtx), vp],
    "sl_moe_down_push": [C.POINTER(N.MoeDownParams), C.POINTER(PushCtx), vp],
    "sl_linear_smallT_bf16_tcgen05_push": [vp, vp, i32, i32, i32, i32, i32, vp, C.POINTER(PushCtx), vp],
})


CollectiveTimeout = N.CollectiveTimeout      # a device-side bounded wait expired (a peer did not publish its flag in time)


class PushSink:
    """Destination of one partial-sum producer: a rotating receive buffer on every rank."""

    def __init__(self, owner: "SymmetricRegion", index: int):
        self.owner = owner
        self.index = index
        self.push = owner.push_ctx[index]
        self.pushed_rows = 0

    def push_tensor(self, x: torch.Tensor) -> "PushSink":
        """Fallback for producers without a fused epilogue: push an fp32 [T, N] tensor."""
        x = x.to(torch.float32).contiguous()
        N.call("sl_push_rows", C.byref(self.push), x.data_ptr(), x.shape[0], x.shape[1], N.stream())
        self.pushed_rows = x.shape[0]
        return self


class BulkSink:
    """Destination of one prefill-sized partial sum [T, H]: row t goes to the staging area of rank t // (T / world).
    `rs` is the view of it that the GEMM epilogue takes, `ctx` the one of the collective kernels."""

    def __init__(self, owner: "SymmetricRegion", lane: int, rows: int):
        self.owner, self.lane, self.rows = owner, lane, rows
        W, H, R = owner.world, owner.row_len, rows // owner.world
        off = owner.lay["bulk"][lane]
        st = owner.bulk_state.data_ptr() + 4 * lane * owner.bulk_words
        self.ctx = BulkCtx(rs_done=st, ag_done=st + 4 * (owner.bulk_rows // 32), status=owner.status_ptr, rank=owner.rank,
                           world=W, slot_rows=R, row_len=H, max_spins=owner.wait_spins)
        self.rs = PushCtx(epoch=0, block_counter=0, rank=owner.rank, world=W, slot_rows=R, row_len=H)
        for r in range(W):
            base = owner.peer_ptrs[r]
            self.ctx.stage[r] = self.rs.bufs[r] = base + off["stage"]
            self.ctx.rs_count[r] = self.rs.flags[r] = base + off["rs_count"]
            self.ctx.full[r] = base + off["full"]
            self.ctx.ag_count[r] = base + off["ag_count"]
        self.pushed_rows = rows

    def push_tensor(self, x: torch.Tensor) -> "BulkSink":
        """Producers without a fused epilogue: send an existing fp32 / bf16 [T, H] tensor to the owners of its rows."""
        if x.dtype not in (torch.float32, torch.bfloat16):
            x = x.to(torch.float32)
        if x.stride(-1) != 1 or x.stride(0) % 8 != 0:
            x = x.contiguous()
        assert x.shape[0] == self.rows and x.shape[1] == self.owner.row_len
        N.call("sl_rs_push_rows", C.byref(self.ctx), x.data_ptr(), x.stride(0), int(x.dtype == torch.float32), N.stream())
        return self


def symmetric_alloc(ctx: ParallelContext, nbytes: int):
    """A zeroed buffer of `nbytes` on every rank, each mapped into every rank's address space.  Returns (this rank's
    tensor, the W addresses at which the ranks' buffers are mapped here, what must stay alive / be closed).  CUDA IPC
    handles travel over the process group; `SLOPLLM_B200_SYMM=torch` uses torch's symmetric-memory rendezvous instead."""
    from ..config import env_str
    if env_str("SYMM") == "torch":
        import torch.distributed._symmetric_memory as symm
        buf = symm.empty(nbytes, dtype=torch.uint8, device=ctx.device)
        buf.zero_()
        hdl = symm.rendezvous(buf, group=ctx.group or dist.group.WORLD)
        return buf, [int(p) for p in hdl.buffer_ptrs], hdl
    buf = torch.zeros(nbytes, dtype=torch.uint8, device=ctx.device)
    torch.cuda.synchronize()
    handle = (C.c_ubyte * 64)()
    offset = C.c_ulonglong(0)
    lib = N.kernels()
    lib.sl_ipc_export.argtypes = [vp, vp, C.POINTER(C.c_ulonglong)]
    lib.sl_ipc_open.argtypes = [vp, C.c_ulonglong, C.POINTER(vp)]
    N.check(lib.sl_ipc_export(buf.data_ptr(), handle, C.byref(offset)), "sl_ipc_export")
    mine = (bytes(handle), int(offset.value))
    everyone = [None] * ctx.world
    dist.all_gather_object(everyone, mine, group=ctx.group)
    ptrs, opened = [], []
    for r, (hb, off) in enumerate(everyone):
        if r == ctx.rank:
            ptrs.append(buf.data_ptr())
            continue
        out = vp()
        hbuf = (C.c_ubyte * 64).from_buffer_copy(hb)
        N.check(lib.sl_ipc_open(hbuf, off, C.byref(out)), f"sl_ipc_open(rank {r})")
        ptrs.append(int(out.value))
        opened.append((int(out.value), int(off)))
    return buf, ptrs, (everyone, opened)


def symmetric_close(keep) -> None:
    """Unmap what `symmetric_alloc` opened (CUDA IPC mappings of the peers' buffers)."""
    if isinstance(keep, tuple) and len(keep) == 2:
        lib = N.kernels()
        lib.sl_ipc_close.argtypes = [vp, C.c_ulonglong]
        for ptr, off in keep[1]:
            lib.sl_ipc_close(ptr, off)


class SymmetricRegion:
    """Symmetric receive buffers + flags, and this rank's local epoch / counter words.

    `peer_ptrs[r]` is the address at which rank r's copy of the region is mapped here.  In tests
    that emulate W ranks on one GPU, W regions are plain allocations on the same device and
    every "rank" gets the same pointer table.
    """

    NUM_BUFS = 3
    BULK_LANES = 3
    GUARD_BYTES = 256
    GUARD_PATTERN = 0xA5

    def __init__(self, rank: int, world: int, slot_rows: int, row_len: int, local: torch.Tensor, peer_ptrs: List[int],
                 gather_bytes: int = 0, cp_shape=None, wait_spins: int = 4_000_000, bulk_rows: int = 0,
                 status: Optional[torch.Tensor] = None):
        assert world <= MAX_RANKS
        self.rank, self.world, self.slot_rows, self.row_len = rank, world, slot_rows, row_len
        self.local = local
        self.peer_ptrs = peer_ptrs
        dev = local.device
        self.state = torch.zeros(64, dtype=torch.int32, device=dev)      # epochs, counters, status
        self.wait_spins = wait_spins
        lay = self.layout(world, slot_rows, row_len, gather_bytes, cp_shape, bulk_rows)
        self.lay = lay
        if local.numel() * local.element_size() < lay["total"]:
            raise ValueError(f"symmetric region of {local.numel() * local.element_size()} bytes is smaller than its layout "
                             f"({lay['total']} bytes): allocate it from SymmetricRegion.layout with the same arguments")
        self.write_canaries()
        # bulk all-reduce lanes: local "blocks past their wait" words, [lane][bulk_rows / 32 group words + 8 source words]
        self.bulk_rows = bulk_rows
        self.bulk_words = bulk_rows // 32 + MAX_RANKS
        self.bulk_state = torch.zeros(max(1, self.BULK_LANES * self.bulk_words), dtype=torch.int32, device=dev)
        st = self.state.data_ptr()
        # {code, site, expected, seen} of an expired wait: words of this region, or (a serving process) the four words of
        # the device's error block that the engine reads back with every step's result
        self.status = status if status is not None else self.state[48:52]
        self.status_ptr = self.status.data_ptr()
        self.push_ctx, self.recv_ctx = [], []
        for b in range(self.NUM_BUFS):
            pc = PushCtx(epoch=st + 4 * b, block_counter=st + 4 * (8 + b), rank=rank, world=world, slot_rows=slot_rows,
                         row_len=row_len)
            for r in range(world):
                pc.bufs[r] = peer_ptrs[r] + lay["data"][b]
                pc.flags[r] = peer_ptrs[r] + lay["flags"][b]
            self.push_ctx.append(pc)
            self.recv_ctx.append(RecvCtx(buf=peer_ptrs[rank] + lay["data"][b], flags=peer_ptrs[rank] + lay["flags"][b],
                                         epoch=st + 4 * b, done_counter=st + 4 * (16 + b), status=self.status_ptr, world=world,
                                         slot_rows=slot_rows, row_len=row_len, max_spins=wait_spins))
        # generic gather (slot 3) and CP merge (slot 4) use their own flags / epochs
        self.gather_ctx = None
        if gather_bytes:
            g = GatherPushCtx(epoch=st + 4 * 3, block_counter=st + 4 * (8 + 3), rank=rank, world=world,
                              slot_bytes=gather_bytes)
            for r in range(world):
                g.bufs[r] = peer_ptrs[r] + lay["gather"]
                g.flags[r] = peer_ptrs[r] + lay["flags"][3]
            self.gather_ctx = g
        self.cp_ctx = None
        if cp_shape is not None:
            Tmax, h, R = cp_shape
            hl = h // world
            cpc = CpPushCtx(epoch=st + 4 * 4, block_counter=st + 4 * (8 + 4), rank=rank, world=world, Tmax=Tmax, h=h, hl=hl, R=R)
            for r in range(world):
                cpc.o_stage[r] = peer_ptrs[r] + lay["cp_o"]
                cpc.lse_stage[r] = peer_ptrs[r] + lay["cp_lse"]
                cpc.flags[r] = peer_ptrs[r] + lay["flags"][4]
            self.cp_ctx = cpc
        self.cp_shape = cp_shape
        self.gather_bytes = gather_bytes

    @classmethod
    def layout(cls, world, slot_rows, row_len, gather_bytes=0, cp_shape=None, bulk_rows=0) -> dict:
        off = 0
        guards = []

        def take(n):
            # every area is followed by a guard zone that no kernel may write (see check_canaries)
            nonlocal off
            o = off
            off += (n + 255) // 256 * 256
            guards.append(off)
            off += cls.GUARD_BYTES
            return o
        lay = {"flags": [take(4 * MAX_RANKS * 2) for _ in range(8)], "data": [], "guards": guards}
        for _ in range(cls.NUM_BUFS):
            lay["data"].append(take(world * slot_rows * row_len * 4))      # {bf16 value, 16-bit tag} per element
        lay["gather"] = take(2 * world * gather_bytes) if gather_bytes else 0          # two halves (epoch parity)
        if cp_shape is not None:
            Tmax, h, R = cp_shape
            hl = h // world
            lay["cp_o"] = take(2 * world * Tmax * hl * R * 4)                          # two halves (epoch parity)
            lay["cp_lse"] = take(2 * world * Tmax * hl * 4)
        lay["bulk"] = []
        if bulk_rows:
            for _ in range(cls.BULK_LANES):                                            # one lane per stream that runs prefill chunks
                lay["bulk"].append({"stage": take(bulk_rows * row_len * 2), "full": take(bulk_rows * row_len * 2),
                                    "rs_count": take(4 * (bulk_rows // 32)), "ag_count": take(4 * MAX_RANKS)})
        lay["total"] = off
        return lay

    def local_view(self, offset: int, nbytes: int) -> torch.Tensor:
        return self.local[offset:offset + nbytes]

    def write_canaries(self) -> None:
        for g in self.lay["guards"]:
            self.local[g:g + self.GUARD_BYTES] = self.GUARD_PATTERN

    def check_canaries(self) -> None:
        """Raise if a guard zone behind one of this rank's areas was written: some kernel (here or on a peer) stored
        past the end of a receive slot, a staging area or a counter array.  Tests call it after every collective test;
        `SLOPLLM_B200_CHECKS=1` makes `check_status` call it after every step (it synchronises)."""
        for i, g in enumerate(self.lay["guards"]):
            zone = self.local[g:g + self.GUARD_BYTES]
            if not bool((zone == self.GUARD_PATTERN).all()):
                bad = int((zone != self.GUARD_PATTERN).nonzero()[0])
                raise RuntimeError(f"rank {self.rank}: guard zone {i} of the symmetric region (offset {g}) was overwritten at byte {bad}")

    def check_status(self) -> None:
        st = self.status.tolist()
        if st[0]:
            self.status.zero_()
            raise CollectiveTimeout(f"rank {self.rank}: device wait expired at site {st[1]} (expected flag {st[2]}, saw {st[3]})")


class NvlinkComm(Comm):
    """Communicator whose hot collectives run inside our kernels over peer memory."""

    MAX_ROWS = 32          # token rows served by the fused decode path; larger steps use the bulk path or NCCL
    BULK_ROWS = 8192       # largest prefill chunk the bulk path takes (two bf16 [BULK_ROWS, H] areas per lane and rank)
    CP_PUSH_ROWS = 8192    # largest step whose context-parallel attention partials are merged through peer memory

    def __init__(self, ctx: ParallelContext, cfg=None, region: Optional[SymmetricRegion] = None):
        super().__init__(ctx)
        self.cfg = cfg
        self._toggle = 0
        self.region = region or self._make_region(ctx, cfg)
        self._lanes = {}       # stream -> bulk lane, in order of first use (the same order on every rank)
        from ..config import env_flag
        self._checks = env_flag("CHECKS")

    @staticmethod
    def bulk_rows_from_env() -> int:
        from ..config import env_flag, env_int
        return env_int("BULK_AR_ROWS", NvlinkComm.BULK_ROWS) if env_flag("BULK_AR") else 0

    @staticmethod
    def _make_region(ctx: ParallelContext, cfg) -> SymmetricRegion:
        """Allocate this rank's region, exchange CUDA IPC handles over the process group and map
        every peer's region (`SLOPLLM_B200_SYMM=torch` uses torch's symmetric-memory rendezvous
        instead)."""
        from ..config import env_str
        H = cfg.hidden_size
        # context parallelism: the attention partials of up to CP_PUSH_ROWS query rows are pushed to the ranks that own their
        # heads (two halves of [world, rows, heads / world, R] fp32 per rank: 2.1 GB at 8 ranks, 8192 rows, 64 heads);
        # larger chunks fall back to the library all-to-all
        from ..config import env_int as _env_int
        cp_rows = max(NvlinkComm.MAX_ROWS, _env_int("CP_PUSH_ROWS", NvlinkComm.CP_PUSH_ROWS))
        cp_shape = (cp_rows, cfg.num_attention_heads, cfg.kv_lora_rank) if ctx.cp else None
        gather_bytes = 1 << 20
        if ctx.cp:
            # the two all-gathers of a context-parallel layer at prefill size: candidate scores [rows, top_k] fp32 and the
            # packed query parts [rows, heads / world, R + rope] bf16 (two halves of `world` slots each: 1.2 GB at 8 ranks)
            hl = max(1, cfg.num_attention_heads // ctx.world)
            per_row = max(4 * cfg.index_topk, 2 * hl * (cfg.kv_lora_rank + cfg.qk_rope_head_dim) + 32)
            gather_bytes = max(gather_bytes, (cp_rows * per_row + 255) // 256 * 256)
        bulk_rows = NvlinkComm.bulk_rows_from_env()
        lay = SymmetricRegion.layout(ctx.world, NvlinkComm.MAX_ROWS, H, gather_bytes, cp_shape, bulk_rows)
        buf, ptrs, keep = symmetric_alloc(ctx, lay["total"])
        torch.cuda.synchronize()
        dist.barrier(group=ctx.group)
        from ..config import env_int
        # bound of every device-side wait, in polls (a poll is 0.03 - 0.3 us; the default is on the order of a second)
        from ..ops import tcgen05
        region = SymmetricRegion(ctx.rank, ctx.world, NvlinkComm.MAX_ROWS, H, buf, ptrs, gather_bytes, cp_shape,
                                 wait_spins=env_int("WAIT_SPINS", 4_000_000), bulk_rows=bulk_rows,
                                 status=tcgen05.error_flag(ctx.device)[12:16])
        region._keep = keep
        return region

    # -- rotation -----------------------------------------------------------------------------
    def begin_forward(self) -> None:
        self._toggle = 0

    def _bulk_sink(self, rows: int) -> Optional[BulkSink]:
        """Bulk lane of the current stream, if this row count can take the bulk path: every rank owns the same number
        of rows, a multiple of 32.  Each stream that runs prefill chunks (the default stream, the two streams of phased
        prefill) gets its own staging areas, because the protocol relies on stream order between consecutive uses."""
        rg = self.region
        if not rg.bulk_rows or rows > rg.bulk_rows or rows % (32 * rg.world) != 0 or rg.row_len % 32 != 0:
            return None
        key = torch.cuda.current_stream(self.ctx.device).cuda_stream if self.ctx.device.type == "cuda" else 0
        lane = self._lanes.get(key)
        if lane is None:
            if len(self._lanes) >= rg.BULK_LANES:
                return None
            lane = self._lanes[key] = len(self._lanes)
        return BulkSink(rg, lane, rows)

    def partial_sink(self, rows: int, final: bool = False):
        if rows > self.MAX_ROWS:
            return self._bulk_sink(rows)
        if final:
            return PushSink(self.region, 2)
        s = PushSink(self.region, self._toggle)
        self._toggle ^= 1
        return s

    # -- bulk all-reduce: owner step and consumer (separate so that a test can run W emulated ranks phase by phase) ----
    def bulk_reduce(self, sink: BulkSink) -> None:
        """Owner step: sum this rank's rows over all ranks' staged partials and store the sums on every rank."""
        N.call("sl_rs_reduce_ag", C.byref(sink.ctx), N.stream())

    def bulk_finish(self, sink: BulkSink, residual, weight, eps):
        """Consumer: wait for every owner's rows, then residual add + RMSNorm.  Returns (normed bf16, residual' fp32)."""
        T, H = sink.rows, self.region.row_len
        out = torch.empty(T, H, dtype=torch.bfloat16, device=self.ctx.device)
        res = torch.empty(T, H, dtype=torch.float32, device=self.ctx.device)
        if residual is not None and (residual.dtype != torch.float32 or not residual.is_contiguous()):
            residual = residual.to(torch.float32).contiguous()
        N.call("sl_bulk_add_rmsnorm", C.byref(sink.ctx), out.data_ptr(), res.data_ptr(), N.ptr(residual), weight.data_ptr(),
               float(eps), N.stream())
        return out, res

    # -- fused all-reduce consumer ----------------------------------------------------------------
    def allreduce_add_rmsnorm(self, ops, partial, residual, weight, eps, want_perm: bool = False):
        if isinstance(partial, BulkSink):
            self.bulk_reduce(partial)
            return self.bulk_finish(partial, residual, weight, eps)
        if not isinstance(partial, PushSink):
            return super().allreduce_add_rmsnorm(ops, partial, residual, weight, eps, want_perm)
        T, H = partial.pushed_rows, self.region.row_len
        dev = self.ctx.device
        out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        res = torch.empty(T, H, dtype=torch.float32, device=dev)
        rc = self.region.recv_ctx[partial.index]
        xp = None
        if want_perm and H % 128 == 0:
            # the consumer of `out` is an NVFP4 tensor-core kernel: write its permuted f16 operand here too
            xp = torch.empty(((T + 7) // 8) * 8 * H, dtype=torch.float16, device=dev)
            out._sl_perm = xp
        N.call("sl_ar_add_rmsnorm", C.byref(rc), out.data_ptr(), res.data_ptr(), N.ptr(residual), weight.data_ptr(), T, H,
               float(eps), N.ptr(xp), N.stream())
        return out, res

    # -- all-gather by peer stores -------------------------------------------------------------------
    def all_gather_list(self, x: torch.Tensor) -> List[torch.Tensor]:
        g = self.region.gather_ctx
        nbytes = x.numel() * x.element_size()
        if g is None or nbytes % 16 != 0 or nbytes > self.region.gather_bytes or self.ctx.world == 1:
            return super().all_gather_list(x)
        x = x.contiguous()
        W, rg = self.ctx.world, self.region
        epoch = rg.state.data_ptr() + 4 * 3
        N.call("sl_gather_push", C.byref(g), x.data_ptr(), nbytes, N.stream())
        N.call("sl_epoch_wait", rg.peer_ptrs[rg.rank] + rg.lay["flags"][3], epoch, W, rg.wait_spins, rg.status_ptr, 4, N.stream())
        out = torch.empty((W,) + tuple(x.shape), dtype=x.dtype, device=x.device)
        N.call("sl_gather_fetch", out.data_ptr(), rg.peer_ptrs[rg.rank] + rg.lay["gather"], epoch, W, rg.gather_bytes, nbytes, N.stream())
        return list(out.unbind(0))

    def all_gather(self, x: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if self.ctx.world == 1:
            return x
        return torch.cat(self.all_gather_list(x), dim=dim)

    # -- context-parallel merge -----------------------------------------------------------------------
    def cp_merge_partials(self, ops, o_part: torch.Tensor, lse_part: torch.Tensor):
        """o_part [T, h, S, R] / lse_part [T, h, S]: this rank's split partials over its KV shard.
        Returns the merged output for this rank's heads, bf16 [T, h/W, R]."""
        rg = self.region
        T, h, S, R = o_part.shape
        W, r = self.ctx.world, self.ctx.rank
        if rg.cp_ctx is None or T > rg.cp_shape[0]:
            o, lse = ops.combine_f32([o_part], [lse_part])
            return super().cp_merge_heads(ops, o, lse)
        # local combine over the splits (fp32 out is needed for the exchange): reuse combine with fp32 via torch
        o, lse = ops.combine_f32([o_part], [lse_part])
        N.call("sl_cp_merge_push", C.byref(rg.cp_ctx), o.data_ptr(), lse.data_ptr(), T, N.stream())
        N.call("sl_epoch_wait", rg.peer_ptrs[r] + rg.lay["flags"][4], rg.state.data_ptr() + 4 * 4, W, rg.wait_spins,
               rg.status_ptr, 5, N.stream())
        Tmax, hl = rg.cp_shape[0], h // W
        stage_o = rg.local_view(rg.lay["cp_o"], W * Tmax * hl * R * 4).view(torch.float32).view(W, Tmax, hl, 1, R)
        stage_l = rg.local_view(rg.lay["cp_lse"], W * Tmax * hl * 4).view(torch.float32).view(W, Tmax, hl, 1)
        # the half of the staging area that this merge used is chosen on the device from the epoch word
        merged, _ = ops.combine([stage_o[i] for i in range(W)], [stage_l[i] for i in range(W)], rows=T, want_lse=False,
                                parity=(rg.state.data_ptr() + 4 * 4, W * Tmax * hl * R, W * Tmax * hl))
        return merged

    def check_status(self) -> None:
        self.region.check_status()
        if self._checks:
            self.region.check_canaries()

    def close(self) -> None:
        """Unmap the peers' regions (CUDA IPC mappings opened by `_make_region`).  Call it when the communicator is
        replaced - after a lost rank its peers' mappings point into a process that no longer exists - with no kernel of
        this communicator in flight."""
        keep = getattr(self.region, "_keep", None)
        if keep is not None:
            symmetric_close(keep)
            self.region._keep = None
