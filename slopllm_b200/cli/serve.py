"""OpenAI-compatible server entry point.

    python -m slopllm_b200.cli.serve --model DIR --mtp --batch-size 8 --port 8000
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m slopllm_b200.cli.serve --model DIR --gpus 0,1,2,3,4,5,6,7

Rank 0 listens; the other ranks follow its scheduler step by step.  Reference:
`src/openai-server.ts:51-103` (flags), `:476-539` (warm-up), `src/main.ts`.
"""
from __future__ import annotations

import argparse
import asyncio
import os
import sys
import time

from .model_cli import add_model_args, build_runtime


BUILTIN_SAMPLING = {"temperature": 0.6, "top_p": 0.95, "top_k": 20, "repetition_penalty": 1.0, "max_tokens": 65536}


def parse_args(argv=None):
    ap = argparse.ArgumentParser(prog="slopllm_b200.cli.serve", description=__doc__.split("\n")[0])
    add_model_args(ap)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--api-key", default=os.environ.get("SLOPLLM_B200_API_KEY") or None,
                    help="bearer token clients must send (default: $SLOPLLM_B200_API_KEY, unset = open)")
    ap.add_argument("--admin-api-key", default=os.environ.get("SLOPLLM_B200_ADMIN_API_KEY") or None)
    ap.add_argument("--served-model-name", default="")
    ap.add_argument("--no-warmup", action="store_true")
    ap.add_argument("--health-port", type=int, default=0, help="multi-rank jobs: port of the heartbeat store (0: no rank-failure monitor)")
    ap.add_argument("--health-timeout", type=float, default=10.0, help="seconds without a heartbeat after which a rank counts as lost")
    ap.add_argument("--dp-port", type=int, default=29640, help="port of the store that carries requests to the other replicas (--dp)")
    # sampling defaults applied when a request does not set them (reference `src/openai-server.ts:51-103`)
    # not given: the checkpoint's generation_config.json / config.json value, else 65536 / 0.6 / 0.95 / 20 / 1.0
    ap.add_argument("--max-tokens", type=int, default=None)
    ap.add_argument("--temperature", type=float, default=None)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--repetition-penalty", type=float, default=None)
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--repetition-penalty-window", type=int, default=64)
    ap.add_argument("--decode-latency", type=float, default=0.0, help="minimum milliseconds per decode step (rate limit)")
    ap.add_argument("--no-mtp", action="store_true", help="ignore --mtp")
    return ap.parse_args(argv)


def warm_up(rt, tokens: int = 32, remote=()) -> float:
    """Requests through the scheduler (and through every remote replica's proxy) before the port opens: one short greedy
    request, then a full batch whose prompts together fill a prefill chunk, so that the first users find the decode graphs
    of batch 1 and of the full batch captured and the allocator already at its serving high-water mark (reference: the
    peak warm-up of `src/openai-server.ts:476-539`).  The prefix caches are flushed afterwards."""
    import threading
    from ..config import SamplingParams
    from ..scheduler.scheduler import GenerationRequest
    t0 = time.time()
    targets = [rt.scheduler, *remote]
    B = max(1, rt.engine_cfg.batch_size)
    per_prompt = max(16, min(1024, rt.engine_cfg.chunk_size // B))
    vocab = getattr(rt.cfg, "vocab_size", 2)
    for round_, (count, plen) in enumerate(((1, 16), (B, per_prompt))):
        if round_ == 1 and B == 1:
            break
        waits = []
        for i, target in enumerate(targets):
            for j in range(count):
                done = threading.Event()
                # different first tokens: the batch must not collapse onto one shared prefix
                ids = [1 + (j * 7 + n) % max(1, vocab - 1) for n in range(plen)]
                target.submit(GenerationRequest(id=f"warmup-{round_}-{i}-{j}", input_ids=ids, max_tokens=tokens,
                                                sampling=SamplingParams(temperature=0.0), on_finish=lambda r, d=done: d.set()))
                waits.append(done)
        for done in waits:
            done.wait(timeout=600)
    for target in targets:
        target.flush_gpu_cache().done.wait(timeout=60)
    return time.time() - t0


def main(argv=None) -> int:
    args = parse_args(argv)
    if args.no_mtp:
        args.mtp = 0
    rt = build_runtime(args)
    from ..config import SamplingParams
    from ..utils.generation_config import apply_generation_defaults
    from ..utils.model_path import resolve_model_path
    origin = apply_generation_defaults(args, resolve_model_path(args.model) if args.model else None, BUILTIN_SAMPLING)
    if any(v == "checkpoint" for v in origin.values()) and rt.ctx.rank == 0 and rt.ctx.dp_rank == 0:
        print("sampling defaults from the checkpoint: " + ", ".join(f"{k}={getattr(args, k)}" for k, v in origin.items()
                                                                    if v == "checkpoint"), file=sys.stderr)
    rt.engine_cfg.max_tokens = args.max_tokens
    rt.engine_cfg.phased_prefill = args.phased_prefill
    rt.engine_cfg.decode_latency_ms = args.decode_latency
    rt.scheduler.decode_latency = args.decode_latency / 1e3
    rt.engine_cfg.sampling = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                                            repetition_penalty=args.repetition_penalty, presence_penalty=args.presence_penalty,
                                            repetition_penalty_window=args.repetition_penalty_window)
    ctx = rt.ctx
    monitor = None
    if args.health_port and (ctx.global_world or ctx.world) > 1:
        # heartbeats of all ranks in a store on job rank 0: a silent rank makes /health answer 503 and the schedulers fail
        # their requests instead of launching collectives that could not complete
        from ..utils.health import HealthMonitor, make_store as make_health_store
        g_rank, g_world = (ctx.global_rank, ctx.global_world) if ctx.global_world else (ctx.rank, ctx.world)
        hstore = make_health_store(g_rank, g_world, port=args.health_port)
        hstore.set(f"ready/{g_rank}", "1")
        hstore.wait([f"ready/{r}" for r in range(g_world)])          # a rank that is still loading is not a dead rank
        monitor = HealthMonitor(hstore, g_rank, g_world, interval_s=0.5, timeout_s=args.health_timeout).start()
        rt.scheduler.health = monitor
    rt.scheduler.start()
    if ctx.rank != 0:
        rt.scheduler._thread.join()              # followers mirror their replica's first rank until it broadcasts stop
        return 0
    front = rt.scheduler
    proxies = []
    if ctx.dp_world > 1:
        # replicas other than the front end's are fed through mailboxes on a store that job rank 0 hosts
        from ..scheduler.data_parallel import DataParallelRouter, ReplicaAgent, ReplicaProxy
        from ..utils.health import make_store
        store = make_store(ctx.global_rank, ctx.global_world, port=args.dp_port)
        if ctx.dp_rank != 0:
            agent = ReplicaAgent(store, ctx.dp_rank, rt.scheduler).start()
            agent._thread.join()                 # until the front end sends "stop"
            rt.scheduler.stop()
            return 0
        proxies = [ReplicaProxy(store, d).start() for d in range(1, ctx.dp_world)]
        front = DataParallelRouter([rt.scheduler] + proxies, page_tokens=rt.engine.kv.tokens_per_page)
    from ..server.openai import OpenAIServer, serve
    if not args.no_warmup:
        print(f"warm-up took {warm_up(rt, remote=proxies):.1f} s", file=sys.stderr)
    name = args.served_model_name or (args.model.rstrip("/").split("/")[-1] if args.model else args.random_init)
    server = OpenAIServer(front, rt.tokenizer, rt.engine_cfg, model_name=name, max_model_len=args.max_model_len,
                          healthy=(monitor.is_healthy if monitor is not None else (lambda: True)),
                          log=lambda line: print(line, file=sys.stderr, flush=True))
    print(f"listening on http://{args.host}:{args.port}  model={name}  ranks={ctx.global_world or ctx.world}  "
          f"replicas={ctx.dp_world}  mtp={args.mtp}", file=sys.stderr)
    import signal

    def _terminate(signum, frame):                       # `docker stop`, `kill`: same orderly exit as Ctrl-C
        raise KeyboardInterrupt
    signal.signal(signal.SIGTERM, _terminate)
    try:
        asyncio.run(serve(server))
    except KeyboardInterrupt:
        print("shutting down: stopping the schedulers of every rank and replica", file=sys.stderr)
    finally:
        for p in proxies:
            p.stop()
        rt.scheduler.stop()
    if ctx.device.type == "cuda":
        # captured graphs still reference the communicators and the symmetric region: leave without the library teardown
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
