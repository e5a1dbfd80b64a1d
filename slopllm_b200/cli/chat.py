"""Interactive chat on the terminal (reference: `src/run_qwen3_unified.ts`): reads a line,
renders the chat template, streams the reply; `/reset` clears the history, `/quit` leaves."""
from __future__ import annotations

import argparse
import sys
import threading

from ..config import SamplingParams
from ..scheduler.scheduler import GenerationRequest
from ..server.parsers import IncrementalDecoder
from .model_cli import add_model_args, build_runtime


def generate(rt, prompt_ids, max_tokens, sampling, out=sys.stdout) -> str:
    detok = IncrementalDecoder(lambda ids: rt.tokenizer.decode(ids, skip_special_tokens=True))
    done = threading.Event()
    pieces = []

    def on_token(t):
        s = detok.push(t)
        if s:
            pieces.append(s)
            out.write(s)
            out.flush()

    req = GenerationRequest(id="chat", input_ids=list(prompt_ids), max_tokens=max_tokens, sampling=sampling, on_token=on_token,
                            on_finish=lambda r: done.set())
    rt.scheduler.submit(req)
    done.wait()
    tail = detok.flush()
    if tail:
        pieces.append(tail)
        out.write(tail)
    out.write("\n")
    return "".join(pieces)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="slopllm_b200.cli.chat")
    add_model_args(ap)
    ap.add_argument("--max-tokens", type=int, default=512)
    # not given: the checkpoint's generation_config.json / config.json value, else 0.6 / 0.95 / 20
    ap.add_argument("--temperature", type=float, default=None)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--prompt", default="", help="answer this one prompt and exit")
    ap.add_argument("--no-thinking", action="store_true")
    args = ap.parse_args(argv)
    rt = build_runtime(args)
    rt.scheduler.start()
    if rt.ctx.rank != 0:
        rt.scheduler._thread.join()
        return 0
    from ..utils.generation_config import apply_generation_defaults
    from ..utils.model_path import resolve_model_path
    args.repetition_penalty = None
    apply_generation_defaults(args, resolve_model_path(args.model) if args.model else None,
                              {"temperature": 0.6, "top_p": 0.95, "top_k": 20, "repetition_penalty": 1.0, "max_tokens": 512})
    sampling = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                              repetition_penalty=args.repetition_penalty)
    history = []
    try:
        while True:
            if args.prompt:
                line = args.prompt
            else:
                try:
                    line = input("> ")
                except EOFError:
                    break
            if line.strip() == "/quit":
                break
            if line.strip() == "/reset":
                history.clear()
                continue
            history.append({"role": "user", "content": line})
            ids = rt.tokenizer.apply_chat_template(history, tokenize=True, add_generation_prompt=True,
                                                   enable_thinking=not args.no_thinking)
            reply = generate(rt, ids, args.max_tokens, sampling)
            history.append({"role": "assistant", "content": reply})
            if args.prompt:
                break
    finally:
        rt.scheduler.stop()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
