"""Communicator factory: in-kernel NVLink collectives when available, library collectives otherwise."""
from __future__ import annotations

from .dist import Comm, ParallelContext


def make_comm(ctx: ParallelContext, cfg=None, fused: bool = True) -> Comm:
    if fused and ctx.world > 1 and ctx.device.type == "cuda":
        from .nvlink import NvlinkComm
        return NvlinkComm(ctx, cfg)
    return Comm(ctx)
