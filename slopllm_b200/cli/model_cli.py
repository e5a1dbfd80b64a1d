"""Shared command-line handling of the entry points: which model, which GPUs, which
parallelism; builds the engine, the sampler, the scheduler and the tokenizer.

Flags follow the reference (`src/model_cli.ts:1-154`, `src/openai-server.ts:51-103`):
`--model --gpus --arena --cp --mtp --batch-size --chunk-size --max-pages --max-host-pages ...`.
One process drives one GPU: start N ranks with
`python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m slopllm_b200.cli.serve ...`;
`--gpus` then only states the expected world size.
"""
from __future__ import annotations

import argparse
import os
from dataclasses import dataclass
from typing import List, Optional

import torch

from ..config import EngineConfig, GlmMoeDsaConfig, env_flag
from ..parallel.dist import ParallelContext, init_from_env


def add_model_args(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--model", default="", help="checkpoint directory or Hugging Face hub id (local cache only)")
    ap.add_argument("--random-init", default="", metavar="SPEC",
                    help="no checkpoint: random weights of 'tiny', 'glm5[:layers]', 'qwen3-tiny' or 'qwen35-tiny'")
    ap.add_argument("--gpus", default="", help="comma-separated device list; its length must equal the number of ranks")
    ap.add_argument("--arena", type=float, default=0.0,
                    help="GiB of device memory this process may allocate per GPU (weights + KV cache + step buffers); a larger "
                         "request fails with an out-of-memory error instead of taking the GPU.  0: no cap")
    ap.add_argument("--cp", action="store_true", help="context parallelism (KV tokens interleaved across ranks)")
    ap.add_argument("--ep", action="store_true", help="expert parallelism for the routed experts")
    ap.add_argument("--dp", type=int, default=1, help="data parallelism: the job's ranks form this many independent model "
                                                      "replicas (each tensor-parallel over ranks / dp GPUs) behind one front end")
    ap.add_argument("--mtp", type=int, nargs="?", const=3, default=0, help="speculative drafts per step (bare flag: 3)")
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--chunk-size", type=int, default=8192)
    ap.add_argument("--max-pages", type=int, default=0, help="KV pages of 64 tokens (0: batch-size * ceil(chunk-size / 64))")
    ap.add_argument("--max-host-pages", type=int, default=0, help="pinned-host prefix tier size in pages (0: off)")
    ap.add_argument("--max-model-len", type=int, default=None,
                    help="longest sequence (prompt + output) a request may reach; default: the checkpoint's "
                         "max_position_embeddings, 65536 without a checkpoint")
    ap.add_argument("--no-cuda-graph", action="store_true")
    ap.add_argument("--phased-prefill", dest="phased_prefill", action="store_true", default=env_flag("PHASED_PREFILL"),
                    help="run large prefill chunks as two halves on two streams (multi-rank jobs); off by default: over "
                         "NVLink the all-reduce is short and two half-size GEMM streams measured slower than one; "
                         "SLOPLLM_B200_PHASED_PREFILL=1 changes the default")
    ap.add_argument("--no-phased-prefill", dest="phased_prefill", action="store_false")
    ap.add_argument("--no-fused-collectives", action="store_true", help="NCCL collectives instead of the in-kernel NVLink ones")
    ap.add_argument("--cpu", action="store_true", help="run on the CPU reference ops (plumbing / debugging)")
    ap.add_argument("--seed", type=int, default=0)


@dataclass
class Runtime:
    cfg: object
    model: object
    engine: object
    scheduler: object
    tokenizer: object
    ctx: ParallelContext
    engine_cfg: EngineConfig
    model_type: str


def _context(args) -> ParallelContext:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    gpus: List[int] = [int(x) for x in args.gpus.split(",") if x != ""] if args.gpus else list(range(world))
    if len(gpus) != world:
        raise SystemExit(f"--gpus names {len(gpus)} devices but the job has {world} rank(s): start one rank per GPU with torchrun")
    dp = max(1, getattr(args, "dp", 1))
    if world % dp != 0:
        raise SystemExit(f"--dp {dp} does not divide the job's {world} rank(s)")
    if world > 1:
        local = int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))
        return init_from_env("gloo" if args.cpu else None, cp=args.cp, ep=args.ep, dp=dp, device_index=gpus[local % len(gpus)])
    dev = torch.device("cpu") if args.cpu or not torch.cuda.is_available() else torch.device("cuda", gpus[0] if gpus else 0)
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
    return ParallelContext(device=dev, cp=args.cp, ep=args.ep)


def arena_fraction(arena_gb: float, total_bytes: int) -> float:
    """Share of the device's memory that `--arena` GiB amounts to (1.0: no cap)."""
    if arena_gb <= 0 or total_bytes <= 0:
        return 1.0
    return min(1.0, arena_gb * (1 << 30) / total_bytes)


def apply_arena_cap(device: torch.device, arena_gb: float) -> float:
    """Cap this process's allocations on `device` at `--arena` GiB (the reference sizes one arena per GPU up front,
    `src/glm_ops.ts:1019-1103`; here the caching allocator gets the same bound).  Returns the fraction applied."""
    if device.type != "cuda":
        return 1.0
    frac = arena_fraction(arena_gb, torch.cuda.get_device_properties(device).total_memory)
    if frac < 1.0:
        torch.cuda.set_per_process_memory_fraction(frac, device)
    return frac


def check_memory_plan(args, ctx: ParallelContext, model_dir: str, model_type: str) -> Optional[str]:
    """Before the weights are read: does this rank's share of the model plus the KV pages asked for fit the memory the
    process may use?  A plan that does not fit is reported on stderr (rank 0) and returned; loading still goes ahead, the
    estimate of the workspace is deliberately generous."""
    if model_type not in ("glm_moe_dsa", "qwen3", "qwen3_5") or ctx.device.type != "cuda":
        return None
    import sys
    from ..utils.sizing import GIB, plan_dense, plan_memory
    total = torch.cuda.get_device_properties(ctx.device).total_memory
    if model_type == "glm_moe_dsa":
        from ..checkpoint.loader import load_config
        p = plan_memory(load_config(model_dir), world=ctx.world, cp=args.cp, ep=args.ep, mtp=args.mtp, batch_size=args.batch_size,
                        chunk_size=args.chunk_size, max_pages=args.max_pages, arena_gb=args.arena, device_gb=total / GIB)
    else:
        import json
        from ..models.dense import DenseConfig
        with open(os.path.join(model_dir, "config.json")) as f:
            dcfg = DenseConfig.from_hf_dict(json.load(f))
        p = plan_dense(dcfg, world=ctx.world, batch_size=args.batch_size, chunk_size=args.chunk_size, max_pages=args.max_pages,
                       arena_gb=args.arena, device_gb=total / GIB)
    if p.requested_fits:
        return None
    msg = (f"memory plan: {p.weights_bytes / GIB:.1f} GiB of weights per rank + about {p.workspace_bytes / GIB:.1f} GiB of "
           f"workspace leave room for {p.max_pages} KV pages, {p.requested_pages} were asked for "
           f"(`python -m slopllm_b200 plan` shows the arithmetic)")
    if ctx.rank == 0 and ctx.dp_rank == 0:
        print(msg, file=sys.stderr)
    return msg


def _random_model(spec: str, ctx: ParallelContext, mtp: int):
    from ..parallel.fused import make_comm
    dtype = torch.bfloat16 if ctx.device.type == "cuda" else torch.float32
    tp_world = ctx.world          # weights stay tensor-parallel under context parallelism too
    tp_rank = ctx.rank if tp_world > 1 else 0
    if spec.startswith("qwen"):
        from ..models.dense import DenseConfig, DenseModel, random_dense_model
        cfg = DenseConfig.tiny(hybrid=spec.startswith("qwen35"))
        w, _ = random_dense_model(cfg, 0, ctx.device, dtype, tp_rank, tp_world)
        return cfg, DenseModel(cfg, w, ctx), cfg.model_type
    from ..models.glm_moe_dsa import GlmMoeDsaModel
    from ..models.weights import random_model
    if spec.startswith("glm5"):
        layers = int(spec.split(":")[1]) if ":" in spec else 78
        cfg = GlmMoeDsaConfig.glm5(num_layers=layers)
        exact = False
    else:
        cfg, exact = GlmMoeDsaConfig.tiny(), True
    w = random_model(cfg, 0, ctx.device, dtype, tp_rank, tp_world, ep=ctx.ep, exact=exact, with_mtp=mtp > 0)
    return cfg, GlmMoeDsaModel(cfg, w, ctx, comm=make_comm(ctx, cfg)), "glm_moe_dsa"


def build_runtime(args, with_scheduler: bool = True) -> Runtime:
    from ..models.registry import inspect_model
    from ..runtime.engine import Engine
    from ..sampling.workspace import SamplingWorkspace
    from ..scheduler.replicated import make_channel
    from ..scheduler.scheduler import GenerationScheduler, HostTier
    from ..server.tokenizer import load_tokenizer
    from ..utils.model_path import resolve_model_path

    ctx = _context(args)
    apply_arena_cap(ctx.device, args.arena)
    if args.no_fused_collectives:
        os.environ["SLOPLLM_B200_FUSED"] = "0"
    model_dir: Optional[str] = None
    if args.random_init:
        cfg, model, model_type = _random_model(args.random_init, ctx, args.mtp)
    else:
        if not args.model:
            raise SystemExit("give --model DIR|HUB_ID or --random-init SPEC")
        model_dir = resolve_model_path(args.model)
        if getattr(args, "max_model_len", None) is None:
            from ..utils.generation_config import max_position_embeddings
            args.max_model_len = max_position_embeddings(model_dir)
        model_type, reg, _ = inspect_model(model_dir, cp=args.cp, mtp=args.mtp)
        check_memory_plan(args, ctx, model_dir, model_type)
        cfg, model = reg.load(model_dir, ctx, args.mtp)
    if getattr(args, "max_model_len", None) is None:
        args.max_model_len = 65536
    ecfg = EngineConfig(model=args.model or args.random_init, gpus=list(range(ctx.world)), arena_gb=args.arena, cp=args.cp, ep=args.ep,
                        mtp=args.mtp, batch_size=args.batch_size, chunk_size=args.chunk_size, max_pages=args.max_pages,
                        max_host_pages=args.max_host_pages, cuda_graph=not args.no_cuda_graph,
                        host=getattr(args, "host", "127.0.0.1"), port=getattr(args, "port", 8000),
                        api_key=getattr(args, "api_key", None), admin_api_key=getattr(args, "admin_api_key", None),
                        fused_collectives=not args.no_fused_collectives)
    vocab = cfg.vocab_size
    sampler = SamplingWorkspace(ctx.device, vocab, seed=args.seed)
    engine = Engine(cfg, model, num_pages=ecfg.max_pages, max_batch=ecfg.batch_size, max_seq_len=args.max_model_len,
                    cuda_graph=ecfg.cuda_graph, mtp=args.mtp, sampler=sampler,
                    phased_prefill=getattr(args, "phased_prefill", False) and ctx.world > 1)
    sched = None
    if with_scheduler:
        eos = list(getattr(cfg, "eos_token_ids", None) or getattr(cfg, "eos_token_id", None) or [])
        tier = None
        if ecfg.max_host_pages > 0 and engine.supports_host_tier():
            tier = HostTier(ecfg.max_host_pages, engine.kv.tokens_per_page, engine.read_page, engine.write_page,
                            read_pages=engine.read_pages, write_pages=engine.write_pages)
        sched = GenerationScheduler(engine, max_batch=ecfg.batch_size, chunk_size=ecfg.chunk_size, eos_token_ids=eos, host_tier=tier,
                                    decode_latency_ms=ecfg.decode_latency_ms, replica_channel=make_channel(ctx))
    tok = load_tokenizer(model_dir, vocab)
    return Runtime(cfg, model, engine, sched, tok, ctx, ecfg, model_type)
