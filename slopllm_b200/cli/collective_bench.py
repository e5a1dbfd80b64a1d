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


def _time_eager(fn, iters: int) -> float:
    """Microseconds per call of `fn` launched eagerly `iters` times (paths that synchronise with the host inside)."""
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) * 1e3 / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def ep_case(args, ctx) -> dict:
    """Expert-parallel MoE layer (256 experts x 2048, top-8, experts split over the ranks) for a chunk of T rows:
    dispatch / grouped FP4 GEMMs / combine through peer memory (`parallel/ep.py`) against the same layer with NCCL
    all-to-all dispatch and combine (host-side counts), and against the dispatch-free form (every rank routes all rows,
    masked partial sums).  Eager launches; the partial sums are compared as they enter the all-reduce that follows."""
    from ..models.glm_moe_dsa import GlmMoeDsaModel
    from ..models.weights import random_model
    from ..parallel.dist import ParallelContext
    ectx = ParallelContext(ctx.rank, ctx.world, ctx.device, False, True, ctx.group)
    cfg = GlmMoeDsaConfig.glm5(num_layers=4)
    w = random_model(cfg, 0, ctx.device, torch.bfloat16, ctx.rank, ctx.world, exact=False, ep=True, with_mtp=False)
    model = GlmMoeDsaModel(cfg, w, ectx, comm=make_comm(ectx, cfg))
    lw = w.layers[3]
    g = torch.Generator(device=ctx.device).manual_seed(5)
    rows = []
    for T in [int(t) for t in args.tokens.split(",") if int(t) >= 33]:
        y = torch.randn(T, cfg.hidden_size, device=ctx.device, generator=g).to(torch.bfloat16)
        if model._ep_exchange_for(lw, y) is None:
            raise RuntimeError("the peer-memory exchange does not take this shape")
        us_f = _time_eager(lambda: model._moe_ep_fused(lw, y), args.iters)
        us_a = _time_eager(lambda: model._moe_ep(lw, y), args.iters)
        us_p = _time_eager(lambda: model._moe_ep_partial(lw, y), args.iters)
        # bytes a rank sends: 4-bit rows + scales of the routes that leave it, bf16 result rows that return
        k, H = cfg.num_experts_per_tok, cfg.hidden_size
        away = (T // ctx.world) * k * (ctx.world - 1) / ctx.world
        nv = away * (H // 2 + H // 16 + 4) + away * H * 2
        flops = 2.0 * (T * k / ctx.world) * 3 * H * cfg.moe_intermediate_size
        roof = max(flops / (args.bf16_tflops * 1e6), nv / (args.nvlink_gbs * 1e3))
        rows.append({"tokens": T, "fused_us": round(us_f, 1), "nccl_all_to_all_us": round(us_a, 1), "masked_partial_us": round(us_p, 1),
                     "speedup_vs_all_to_all": round(us_a / us_f, 2), "roofline_us": round(roof, 1),
                     "fused_fraction_of_roofline": round(roof / us_f, 3), "nvlink_bytes_out_per_rank": int(nv)})
    model._ep_exchange.check_status() if getattr(model, "_ep_exchange", None) is not None else None
    return {"op": "EP MoE layer: dispatch + grouped FP4 GEMMs + combine", "world": ctx.world, "rows": rows}


def cp_case(args, ctx) -> dict:
    """Context-parallel attention merge for B decode rows: every rank's partial (o, lse) over its KV shard, 64 heads x 512
    latent values, pushed to the ranks that own the heads and merged by log-sum-exp there (`sl_cp_merge_push` + combine)
    against all-to-all + merge through NCCL."""
    from ..ops.cuda_ops import CudaOps
    from ..parallel.dist import ParallelContext
    cctx = ParallelContext(ctx.rank, ctx.world, ctx.device, True, False, ctx.group)
    cfg = GlmMoeDsaConfig.glm5(num_layers=4)
    ops = CudaOps(cfg, cctx)
    fused, plain = make_comm(cctx, cfg), Comm(cctx)
    h, R = cfg.num_attention_heads, cfg.kv_lora_rank
    g = torch.Generator(device=ctx.device).manual_seed(ctx.rank + 9)
    rows = []
    for B in (1, 8, 32, 64):
        o = torch.randn(B, h, 1, R, device=ctx.device, generator=g)
        lse = torch.randn(B, h, 1, device=ctx.device, generator=g)
        us_f = _time_graph(lambda: fused.cp_merge_partials(ops, o, lse), args.iters)
        us_l = _time_graph(lambda: plain.cp_merge_heads(ops, o[:, :, 0], lse[:, :, 0]), args.iters)
        nv = B * h * (R + 1) * 4 * (ctx.world - 1) / ctx.world
        roof = nv / (args.nvlink_gbs * 1e3)
        rows.append({"rows": B, "fused_us": round(us_f, 2), "library_us": round(us_l, 2), "speedup": round(us_l / us_f, 2),
                     "roofline_us": round(roof, 3), "fused_fraction_of_roofline": round(roof / us_f, 3)})
    fused.check_status() if hasattr(fused, "check_status") else None
    return {"op": "CP attention merge (push + log-sum-exp combine)", "world": ctx.world, "heads": h, "R": R, "rows": rows}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="slopllm_b200.cli.collective_bench")
    ap.add_argument("--cases", default="oproj", help="comma-separated: oproj (GEMM + all-reduce), ep (expert-parallel MoE layer), cp (attention merge)")
    ap.add_argument("--tokens", default="1,8,32")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--hbm-gbs", type=float, default=6550.0, help="measured copy bandwidth used as the HBM roofline")
    ap.add_argument("--nvlink-gbs", type=float, default=770.0, help="measured peer copy bandwidth per direction")
    ap.add_argument("--bf16-tflops", type=float, default=1590.0, help="measured bf16 GEMM throughput (tensor roofline of large T)")
    args = ap.parse_args(argv)
    ctx = init_from_env()
    W, dev = ctx.world, ctx.device
    cases = set(args.cases.split(","))
    for name, fn in (("cp", cp_case), ("ep", ep_case)):
        if name in cases:
            out = fn(args, ctx)
            if ctx.rank == 0:
                print(json.dumps(out), flush=True)
            dist.barrier()
    if "oproj" not in cases:
        dist.barrier()
        os._exit(0)
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
            push_bytes = T * H * 4 * (W - 1)                       # 4-byte {bf16, tag} words to every peer
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
