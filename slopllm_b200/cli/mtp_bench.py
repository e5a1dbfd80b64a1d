"""MTP decode benchmark: steps/s, tokens/s and accept-length statistics for a batch of sequences
(reference: `src/run_glm51_multiple_mtp.ts`; its `--profile` flag brackets the timed region with
the CUDA profiler API so that an external profiler captures only those steps)."""
from __future__ import annotations

import argparse
import json

import torch

from ..utils.mtp_stats import MtpStats
from .common_bench import synthetic_prompt, timed_ms
from .model_cli import add_model_args, build_runtime


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="slopllm_b200.cli.mtp_bench")
    add_model_args(ap)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--profile", action="store_true")
    args = ap.parse_args(argv)
    if args.mtp <= 0:
        args.mtp = 3
    rt = build_runtime(args, with_scheduler=False)
    eng, B = rt.engine, args.batch_size
    seqs = [eng.kv.new_sequence() for _ in range(B)]
    prompts = [synthetic_prompt(rt.cfg.vocab_size, args.context, seed=b) for b in range(B)]
    last, hid = eng.prefill(seqs, prompts, chunk_size=args.chunk_size, want_hidden=True)
    seed = eng.mtp_seed(seqs, last, hid)
    stats = MtpStats(args.mtp)
    for _ in range(args.warmup):
        _, last, seed = eng.mtp_decode_step(seqs, last, seed)

    def run():
        nonlocal last, seed
        for _ in range(args.steps):
            acc, last, seed = eng.mtp_decode_step(seqs, last, seed)
            stats.record(acc)

    cuda = rt.ctx.device.type == "cuda"
    if args.profile and cuda:
        torch.cuda.cudart().cudaProfilerStart()
    ms = timed_ms(rt.ctx, run)
    if args.profile and cuda:
        torch.cuda.cudart().cudaProfilerStop()
    if rt.ctx.rank == 0:
        out = stats.summary()
        out.update({"batch": B, "context": args.context, "ms_per_step": ms / args.steps, "steps_s": args.steps * 1e3 / ms,
                    "sequence_steps_s": B * args.steps * 1e3 / ms, "tok_s": stats.accepted_tokens * 1e3 / ms, "ranks": rt.ctx.world})
        print(json.dumps(out), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
