"""Batch x context sweep of decode step time (reference: `src/run_sweep.ts`): for each context
length the KV cache is filled by prefill, then `--steps` decode steps are timed per batch size."""
from __future__ import annotations

import argparse
import json

from .common_bench import synthetic_prompt, timed_ms
from .model_cli import add_model_args, build_runtime


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="slopllm_b200.cli.sweep")
    add_model_args(ap)
    ap.add_argument("--batches", default="1,2,4,8")
    ap.add_argument("--contexts", default="1024,8192")
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args(argv)
    batches = [int(x) for x in args.batches.split(",")]
    args.batch_size = max(args.batch_size, max(batches))
    rt = build_runtime(args, with_scheduler=False)
    eng = rt.engine
    for ctx_len in [int(x) for x in args.contexts.split(",")]:
        for B in batches:
            seqs = [eng.kv.new_sequence() for _ in range(B)]
            prompts = [synthetic_prompt(rt.cfg.vocab_size, ctx_len, seed=b) for b in range(B)]
            last, _ = eng.prefill(seqs, prompts, chunk_size=args.chunk_size)
            for _ in range(args.warmup):
                last = eng.decode_step(seqs, last)

            def run():
                nonlocal last
                for _ in range(args.steps):
                    last = eng.decode_step(seqs, last)

            ms = timed_ms(rt.ctx, run) / args.steps
            for s in seqs:
                eng.kv.free_sequence(s)
                eng.release(s)
            if rt.ctx.rank == 0:
                print(json.dumps({"context": ctx_len, "batch": B, "ms_per_step": ms, "tok_s": B * 1e3 / ms, "ranks": rt.ctx.world}),
                      flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
