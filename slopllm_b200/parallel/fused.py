"""Communicator factory: in-kernel NVLink collectives when available, library collectives otherwise."""
from __future__ import annotations

from .dist import Comm, ParallelContext


def make_comm(ctx: ParallelContext, cfg=None, fused: bool = True) -> Comm:
    """`fused=False`, `--no-fused-collectives` or `SLOPLLM_B200_FUSED=0` select the library collectives (the reference's
    `SLOPLLM_DISABLE_P2P_ALLREDUCE`, `src/parallel_ops.ts:2458`)."""
    from ..config import env_flag
    if fused and env_flag("FUSED", True) and ctx.world > 1 and ctx.device.type == "cuda":
        from .nvlink import NvlinkComm
        return NvlinkComm(ctx, cfg)
    return Comm(ctx)
