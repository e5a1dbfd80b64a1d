"""Prefill throughput / time-to-first-token at a list of context lengths
(reference: `src/run_prefill_benchmark.ts`).  Prints one JSON line per context on rank 0."""
from __future__ import annotations

import argparse
import json

from .common_bench import synthetic_prompt, timed_ms
from .model_cli import add_model_args, build_runtime


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="slopllm_b200.cli.prefill_bench")
    add_model_args(ap)
    ap.add_argument("--contexts", default="8192", help="comma-separated prompt lengths")
    ap.add_argument("--repeats", type=int, default=1)
    args = ap.parse_args(argv)
    rt = build_runtime(args, with_scheduler=False)
    eng = rt.engine
    for n in [int(x) for x in args.contexts.split(",")]:
        best = None
        for rep in range(args.repeats):
            prompt = synthetic_prompt(rt.cfg.vocab_size, n, seed=rep)
            s = eng.kv.new_sequence()
            ms = timed_ms(rt.ctx, lambda: eng.prefill([s], [prompt], chunk_size=args.chunk_size))
            eng.kv.free_sequence(s)
            eng.release(s)
            eng.check_device_errors()
            best = ms if best is None else min(best, ms)
        if rt.ctx.rank == 0:
            print(json.dumps({"context": n, "ttft_s": best / 1e3, "prefill_tok_s": n / (best / 1e3), "chunk_size": args.chunk_size,
                              "ranks": rt.ctx.world, "cp": args.cp}), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
