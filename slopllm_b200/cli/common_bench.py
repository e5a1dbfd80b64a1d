"""Helpers shared by the benchmark / evaluation entry points: device-timed regions, rank-max
reduction, synthetic prompts."""
from __future__ import annotations

import time
from typing import Callable, List

import torch


def sync(ctx) -> None:
    if ctx.device.type == "cuda":
        torch.cuda.synchronize(ctx.device)
    if ctx.world > 1:
        import torch.distributed as dist
        dist.barrier()


def timed_ms(ctx, fn: Callable[[], object]) -> float:
    """Milliseconds of `fn` on the device (CUDA events) or the host clock on CPU; max over ranks."""
    sync(ctx)
    if ctx.device.type == "cuda":
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize(ctx.device)
        ms = a.elapsed_time(b)
    else:
        t0 = time.perf_counter()
        fn()
        ms = (time.perf_counter() - t0) * 1e3
    if ctx.world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], dtype=torch.float64, device=ctx.device if ctx.device.type == "cuda" else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    return ms


def synthetic_prompt(vocab: int, n: int, seed: int = 0) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(2, max(3, vocab - 1), (n,), generator=g).tolist()
