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
    ap.add_argument("--op-times", action="store_true",
                    help="CUDA-event pair around every backend op and every collective of the last repeat; rank 0 prints the breakdown")
    args = ap.parse_args(argv)
    rt = build_runtime(args, with_scheduler=False)
    eng = rt.engine
    timers = None
    if args.op_times:
        from ..utils.tracing import OpTimers
        timers = OpTimers(eng.model.ops)
        comm = eng.model.comm
        timers.attach(comm, [n for n in ("allreduce_add_rmsnorm", "all_gather", "all_gather_many", "all_gather_list", "cp_merge_topk",
                                         "cp_merge_partials", "cp_merge_heads", "all_to_all") if hasattr(comm, n)], prefix="comm.")
    for n in [int(x) for x in args.contexts.split(",")]:
        best = None
        for rep in range(args.repeats):
            prompt = synthetic_prompt(rt.cfg.vocab_size, n, seed=rep)
            s = eng.kv.new_sequence()
            if timers is not None:
                timers.reset()
            ms = timed_ms(rt.ctx, lambda: eng.prefill([s], [prompt], chunk_size=args.chunk_size))
            eng.kv.free_sequence(s)
            eng.release(s)
            eng.check_device_errors()
            best = ms if best is None else min(best, ms)
        if rt.ctx.rank == 0:
            print(json.dumps({"context": n, "ttft_s": best / 1e3, "prefill_tok_s": n / (best / 1e3), "chunk_size": args.chunk_size,
                              "ranks": rt.ctx.world, "cp": args.cp}), flush=True)
        if timers is not None:
            rows = timers.summary()
            if rt.ctx.rank == 0:
                print(json.dumps({"context": n, "op_times": rows}), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
