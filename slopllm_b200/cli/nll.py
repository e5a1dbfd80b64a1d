"""Teacher-forced negative log-likelihood / perplexity of a token file or text
(reference: `src/run_nll.ts`).  The text is cut into windows of `--window` tokens, each is
prefilled with all-token logits and scored against its shifted self."""
from __future__ import annotations

import argparse
import json
import math

import torch

from ..ops import reference as R
from .model_cli import add_model_args, build_runtime


def score_window(rt, ids):
    """Sum of -log p(ids[i+1] | ids[:i+1]) over the window and the number of scored tokens."""
    eng = rt.engine
    s = eng.kv.new_sequence()
    eng.kv.append_tokens(s, ids)
    st = eng._eager_state(ids, list(range(len(ids))), [0] * len(ids), [s], max_kv_len=len(ids))
    eng._prepare(st, [s])
    hidden = rt.model.forward_hidden(st, eng.cache)
    logits = rt.model.compute_logits(hidden[:-1]).to(torch.float32)
    nll = R.log_softmax_nll(logits, torch.tensor(ids[1:], device=logits.device)).sum().item()
    eng.kv.free_sequence(s)
    eng.release(s)
    return nll, len(ids) - 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="slopllm_b200.cli.nll")
    add_model_args(ap)
    ap.add_argument("--text-file", default="", help="UTF-8 text to tokenise and score")
    ap.add_argument("--ids-file", default="", help="JSON list of token ids to score")
    ap.add_argument("--window", type=int, default=2048)
    args = ap.parse_args(argv)
    rt = build_runtime(args, with_scheduler=False)
    if args.ids_file:
        with open(args.ids_file) as f:
            ids = json.load(f)
    elif args.text_file:
        with open(args.text_file, encoding="utf-8") as f:
            ids = rt.tokenizer.encode(f.read())
    else:
        raise SystemExit("give --text-file or --ids-file")
    total, count = 0.0, 0
    for lo in range(0, len(ids) - 1, args.window):
        w = ids[lo:lo + args.window + 1]
        if len(w) < 2:
            break
        nll, n = score_window(rt, w)
        total, count = total + nll, count + n
    if rt.ctx.rank == 0:
        print(json.dumps({"tokens": count, "nll": total / max(1, count), "ppl": math.exp(total / max(1, count))}), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
