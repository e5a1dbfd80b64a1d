"""Op-level comparison of the fused compute + all-reduce path with the library path on real
peer memory (one rank per GPU under torchrun):

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m slopllm_b200.cli.collective_bench

For each token count T it times, with CUDA events on the launching stream and the max over
ranks, a captured graph of `--iters` repetitions of
    fused:   o_proj GEMM whose epilogue stores fp32 partial rows into every rank's receive slot
             + the consumer kernel (wait for flags, sum slots, residual add, RMSNorm)
    library: the same GEMM writing locally + NCCL all-reduce + the fused add+RMSNorm kernel
and reports microseconds per repetition next to the roofline time of the op: the slower of
weight bytes / measured HBM bandwidth and pushed bytes / NVLink bandwidth per direction.
Token counts above 32 (e.g. `--tokens 4096,8192` with `SLOPLLM_B200_BULK_AR=1`) compare the bulk path - reduce-scatter
from the GEMM epilogue, owner reduce + all-gather push, wait + add + RMSNorm - with GEMM + NCCL + add + RMSNorm; its
roofline is the slower of FLOPs / measured bf16 GEMM throughput and 2 (W-1)/W T H 2 bytes / NVLink bandwidth.
Shapes are GLM-5 class at TP = world: K = 64 * 256 / world, N = hidden 6144, NVFP4 weights.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..config import GlmMoeDsaConfig
from ..models.weights import random_layer
from ..parallel.dist import Comm, init_from_env
from ..parallel.fused import make_comm


def _time_graph(fn, iters: int, reps: int = 5) -> float:
    """Capture `iters` calls of fn in one graph, replay it `reps` times, return microseconds per call."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(iters):
            fn()
    g.replay()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) * 1e3 / (reps * iters)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="slopllm_b200.cli.collective_bench")
    ap.add_argument("--tokens", default="1,8,32")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--hbm-gbs", type=float, default=6550.0, help="measured copy bandwidth used as the HBM roofline")
    ap.add_argument("--nvlink-gbs", type=float, default=770.0, help="measured peer copy bandwidth per direction")
    ap.add_argument("--bf16-tflops", type=float, default=1590.0, help="measured bf16 GEMM throughput (tensor roofline of large T)")
    args = ap.parse_args(argv)
    ctx = init_from_env()
    W, dev = ctx.world, ctx.device
    cfg = GlmMoeDsaConfig.glm5(num_layers=4)
    H = cfg.hidden_size
    from ..ops.cuda_ops import CudaOps
    ops = CudaOps(cfg, ctx)
    fused, plain = make_comm(ctx, cfg), Comm(ctx)
    lw = random_layer(cfg, 3, 0, dev, torch.bfloat16, tp_rank=ctx.rank, tp_world=W, exact=False)
    K = lw.o_proj.in_features
    g = torch.Generator(device=dev).manual_seed(ctx.rank)
    rows = []
    if hasattr(fused, "begin_forward"):
        fused.begin_forward()
    for T in [int(t) for t in args.tokens.split(",")]:
        x = torch.randn(T, K, device=dev, generator=g).to(torch.bfloat16)
        res = torch.zeros(T, H, device=dev)

        def run_fused():
            # consecutive uses alternate between two receive buffers, as inside a forward pass
            s = ops.linear(x, lw.o_proj, out_f32=True, sink=fused.partial_sink(T))
            return fused.allreduce_add_rmsnorm(ops, s, res, lw.post_attn_norm, cfg.rms_norm_eps)

        def run_lib():
            y = ops.linear(x, lw.o_proj, out_f32=True)
            return plain.allreduce_add_rmsnorm(ops, y, res, lw.post_attn_norm, cfg.rms_norm_eps)

        us_f = _time_graph(run_fused, args.iters)
        us_l = _time_graph(run_lib, args.iters)
        weight_bytes = H * K // 2 + H * K // 16
        if T <= 32:
            push_bytes = T * H * 4 * (W - 1)                       # fp32 rows to every peer
            roof_us = max(weight_bytes / (args.hbm_gbs * 1e3), push_bytes / (args.nvlink_gbs * 1e3))
        else:
            push_bytes = 2 * (W - 1) * (T // W) * H * 2            # bf16: partial rows to their owners, sums to every peer
            roof_us = max(2.0 * T * H * K / (args.bf16_tflops * 1e6), push_bytes / (args.nvlink_gbs * 1e3))
        rows.append({"tokens": T, "fused_us": round(us_f, 2), "library_us": round(us_l, 2), "speedup": round(us_l / us_f, 2),
                     "roofline_us": round(roof_us, 2), "fused_fraction_of_roofline": round(roof_us / us_f, 3),
                     "weight_bytes": weight_bytes, "nvlink_bytes_out_per_rank": push_bytes})
    fused.check_status() if hasattr(fused, "check_status") else None
    if ctx.rank == 0:
        print(json.dumps({"op": "o_proj NVFP4 GEMM + all-reduce + add + RMSNorm", "world": W, "K": K, "N": H, "rows": rows}), flush=True)
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    raise SystemExit(main())
