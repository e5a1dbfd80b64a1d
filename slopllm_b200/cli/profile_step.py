"""Run decode steps of ONE rank's shard of a GLM-5-class model on one GPU, without collectives,
for kernel profiling and per-rank timing.

    python -m slopllm_b200.cli.profile_step --batch 8 --context 3000 --tp-shape 8 --layers 5 --steps 3
        eager launches (one kernel per op) for a profiler's launch list / counter capture
    python -m slopllm_b200.cli.profile_step --batch 8 --context 4096 --tp-shape 8 --layers 78 --timed 30
        CUDA-graph replay timed with CUDA events: the per-rank kernel chain of a TP-8 step

    python -m slopllm_b200.cli.profile_step --batch 1 --context 4096 --tp-shape 8 --layers 78 --mtp 3 --timed 20
        speculative steps (3 drafts + verification + reseed) instead of plain decode steps; without --timed they run eagerly

    python -m slopllm_b200.cli.profile_step --prefill 2048 --tp-shape 8 --layers 5
        one eager prefill chunk (tcgen05 GEMMs, grouped expert GEMMs, prefill attention / indexer)
    python -m slopllm_b200.cli.profile_step --prefill 4096 --tp-shape 8 --layers 6 --op-times
        the same chunk with a CUDA-event pair around every backend op (device time per op, no profiler)
    python -m slopllm_b200.cli.profile_step --prefill 4096 --context 65536 --tp-shape 8 --layers 6 --op-times
        a chunk that extends a sequence with 65536 cached tokens (the indexer scans all of them)
    python -m slopllm_b200.cli.profile_step --fused-emulated 8 --batch 8
        the fused GEMM + all-reduce kernels at production shapes with all "ranks" in this process: every rank's
        producer kernel stores into the receive slots of all ranks (here all on one GPU), then each rank's consumer
        reduces.  Producers never wait; consumers run after every producer has been launched.

`--tp-shape N` builds rank 0's 1/N shard (the shapes every rank of a TP-N job runs); results of the
collectives are not needed for timing, so the numerics are those of a partial sum.
The KV / indexer caches are filled with valid packed rows so that attention sees `--context` keys.
"""
from __future__ import annotations

import argparse
import json

import torch

from ..config import GlmMoeDsaConfig
from ..models.glm_moe_dsa import GlmMoeDsaModel
from ..models.weights import random_model
from ..ops import quant
from ..parallel.dist import ParallelContext
from ..runtime.engine import Engine


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="slopllm_b200.cli.profile_step")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--context", type=int, default=None, help="cached tokens per sequence (decode default 3000, prefill default 0)")
    ap.add_argument("--tp-shape", type=int, default=1)
    ap.add_argument("--layers", type=int, default=5, help="3 dense + MoE layers (layer 3 has a full indexer, layer 4 shares it)")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--timed", type=int, default=0, help="time this many graph-replayed steps instead of running eager steps")
    ap.add_argument("--mtp", type=int, default=0)
    ap.add_argument("--prefill", type=int, default=0, help="run one eager prefill chunk of this many tokens instead of decode steps")
    ap.add_argument("--op-times", action="store_true", help="eager run with a CUDA-event pair around every backend op; prints the breakdown")
    ap.add_argument("--fused-emulated", type=int, default=0, metavar="W", help="fused GEMM+all-reduce kernels with W emulated ranks")
    args = ap.parse_args(argv)
    if args.context is None:
        args.context = 0 if args.prefill > 0 else 3000
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if args.fused_emulated:
        return fused_emulated(args, dev)
    cfg = GlmMoeDsaConfig.glm5(num_layers=args.layers)
    w = random_model(cfg, 0, dev, torch.bfloat16, 0, args.tp_shape, exact=False, with_mtp=args.mtp > 0)
    B = args.batch
    pages = (args.prefill + args.context) // 64 + 8 if args.prefill > 0 else B * (args.context // 64 + 8) + 8
    eng = Engine(cfg, GlmMoeDsaModel(cfg, w, ParallelContext(device=dev)), num_pages=pages, max_batch=B,
                 max_seq_len=args.context + args.prefill + 1024, cuda_graph=args.timed > 0, mtp=args.mtp)
    seqs = [eng.kv.new_sequence() for _ in range(B)] if args.prefill <= 0 else []
    for s in seqs:
        eng.kv.append_tokens(s, [1] * args.context)
        eng.kv.report_tokens(s)
    for lc in eng.cache.layers:
        n = lc.kv.shape[0]
        lc.kv.copy_(quant.pack_kv_rows(torch.randn(n, cfg.kv_lora_rank, device=dev), torch.randn(n, cfg.qk_rope_head_dim, device=dev)))
        if lc.idx is not None:
            lc.idx.copy_(quant.pack_index_rows(torch.randn(n, cfg.index_head_dim, device=dev)))
    last = [5] * B
    timers = None
    if args.op_times:
        from ..utils.tracing import OpTimers
        timers = OpTimers(eng.model.ops)
    if args.prefill > 0:
        s = eng.kv.new_sequence()
        if args.context > 0:                    # the chunk extends a sequence whose first `context` tokens are cached
            eng.kv.append_tokens(s, [1] * args.context)
            eng.kv.report_tokens(s)
        prompt = torch.randint(2, cfg.vocab_size - 1, (args.prefill,), generator=torch.Generator().manual_seed(0)).tolist()
        for i in range(2):                      # second pass re-uses the allocator's blocks (steady state)
            if timers is not None:
                timers.reset()
            toks, _ = eng.prefill([s], [[1] * args.context + prompt], chunk_size=args.prefill)
            eng.kv.truncate(s, args.context)
        torch.cuda.synchronize()
        out = {"mode": "prefill", "tokens": args.prefill, "next": toks}
        if timers is not None:
            out["op_times"] = timers.summary()
        print(json.dumps(out))
        return 0
    if args.mtp > 0:
        # speculative steps: D drafts from the MTP layer, one verification pass of the main model, reseed
        hs = [torch.zeros(1, cfg.hidden_size, dtype=torch.bfloat16, device=dev) for _ in seqs]
        seed = eng.mtp_seed(seqs, last, hs)
        n = args.timed if args.timed > 0 else args.steps
        for _ in range(5 if args.timed > 0 else 0):
            _, last, seed = eng.mtp_decode_step(seqs, last, seed)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n):
            if timers is not None and i == n - 1:
                timers.reset()
            _, last, seed = eng.mtp_decode_step(seqs, last, seed)
        b.record()
        torch.cuda.synchronize()
        out = {"mode": "mtp-graph" if args.timed > 0 else "mtp-eager", "mtp": args.mtp, "batch": B, "steps": n,
               "ms_per_step": a.elapsed_time(b) / n, "last": last}
        if timers is not None:
            out["op_times"] = timers.summary()
        print(json.dumps(out))
        return 0
    if args.timed <= 0:
        for i in range(args.steps):
            if timers is not None and i == args.steps - 1:
                timers.reset()                  # keep the last (warm) step only
            torch.cuda.nvtx.range_push(f"decode_step_{i}")
            last = eng.decode_step(seqs, last)
            torch.cuda.nvtx.range_pop()
        torch.cuda.synchronize()
        out = {"mode": "eager", "steps": args.steps, "last": last}
        if timers is not None:
            out["op_times"] = timers.summary()
        print(json.dumps(out))
        return 0
    for _ in range(5):
        last = eng.decode_step(seqs, last)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.timed):
        last = eng.decode_step(seqs, last)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.timed
    print(json.dumps({"mode": "graph", "batch": B, "context": args.context, "tp_shape": args.tp_shape, "layers": args.layers,
                      "ms_per_step": ms, "us_per_layer": 1e3 * ms / args.layers}))
    return 0


def fused_emulated(args, dev) -> int:
    """o_proj (NVFP4, K = 64 heads * 256 / W) and the MoE layer with their all-reduce fused in, W ranks emulated."""
    from ..models.weights import random_layer
    from ..ops.cuda_ops import CudaOps
    from ..parallel.nvlink import NvlinkComm, SymmetricRegion
    W, T = args.fused_emulated, args.batch
    cfg = GlmMoeDsaConfig.glm5(num_layers=4)
    H = cfg.hidden_size
    lay = SymmetricRegion.layout(W, 32, H, 0, None)
    bufs = [torch.zeros(lay["total"], dtype=torch.uint8, device=dev) for _ in range(W)]
    ptrs = [b.data_ptr() for b in bufs]
    regions = [SymmetricRegion(r, W, 32, H, bufs[r], ptrs) for r in range(W)]
    comms = [NvlinkComm(ParallelContext(r, W, dev), cfg, region=regions[r]) for r in range(W)]
    ops = CudaOps(cfg)
    lws = [random_layer(cfg, 3, 0, dev, torch.bfloat16, tp_rank=r, tp_world=W, exact=False) for r in range(W)]
    g = torch.Generator(device=dev).manual_seed(0)
    x_attn = torch.randn(T, lws[0].o_proj.in_features, device=dev, generator=g).to(torch.bfloat16)
    x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    res = torch.zeros(T, H, device=dev)
    for it in range(args.steps):
        for r in range(W):
            comms[r].begin_forward()
        sinks = [ops.linear(x_attn, lws[r].o_proj, out_f32=True, sink=comms[r].partial_sink(T)) for r in range(W)]
        outs = [comms[r].allreduce_add_rmsnorm(ops, sinks[r], res, lws[r].post_attn_norm, cfg.rms_norm_eps) for r in range(W)]
        sinks = [ops.moe_tp(x, lws[r], sink=comms[r].partial_sink(T, final=True)) for r in range(W)]
        outs = [comms[r].allreduce_add_rmsnorm(ops, sinks[r], res, lws[r].input_norm, cfg.rms_norm_eps) for r in range(W)]
    torch.cuda.synchronize()
    for c in comms:
        c.check_status()
    print(json.dumps({"mode": "fused-emulated", "ranks": W, "tokens": T, "checksum": float(outs[0][0].float().abs().sum())}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
