"""Memory plan of a deployment before anything is loaded:

    python -m slopllm_b200 plan --model <dir> --world 8 --cp --mtp 3 --chunk-size 8192 --max-pages 8192 [--arena 160]
    python -m slopllm_b200 plan --random-init glm5 --world 8

prints the per-rank weight bytes under the chosen parallelism, the cost of a KV page, an estimate of a prefill chunk's
workspace, how many pages (and tokens of context) fit in the memory the process may use, and whether the pages asked for
fit.  Nothing is allocated and no GPU is needed (`utils/sizing.py`); the last line is the plan as JSON.
"""
from __future__ import annotations

import argparse
import json

from ..config import GlmMoeDsaConfig
from ..utils.sizing import GIB, plan_memory


def _config(args) -> GlmMoeDsaConfig:
    if args.model:
        from ..checkpoint.loader import load_config
        from ..models.registry import inspect_model
        from ..utils.model_path import resolve_model_path
        model_dir = resolve_model_path(args.model)
        model_type, _, raw = inspect_model(model_dir)
        if model_type in ("qwen3", "qwen3_5"):
            from ..models.dense import DenseConfig
            return DenseConfig.from_hf_dict(raw)
        if model_type != "glm_moe_dsa":
            raise SystemExit(f"plan: the sizing arithmetic covers glm_moe_dsa, qwen3 and qwen3_5; {args.model} is {model_type}")
        return load_config(model_dir)
    spec = args.random_init or "glm5"
    if spec.startswith("qwen"):
        from ..models.dense import DenseConfig
        return DenseConfig.tiny(hybrid=spec.startswith("qwen35"))
    if spec.startswith("glm5"):
        return GlmMoeDsaConfig.glm5(num_layers=int(spec.split(":")[1]) if ":" in spec else 78)
    return GlmMoeDsaConfig.tiny()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="slopllm_b200.cli.plan", description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="", help="checkpoint directory or hub id (only config.json is read)")
    ap.add_argument("--random-init", default="", help="glm5[:layers], tiny, qwen3 or qwen35 instead of a checkpoint")
    ap.add_argument("--world", type=int, default=1, help="GPUs of one replica")
    ap.add_argument("--cp", action="store_true")
    ap.add_argument("--ep", action="store_true")
    ap.add_argument("--mtp", type=int, nargs="?", const=3, default=0)
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--chunk-size", type=int, default=8192)
    ap.add_argument("--max-pages", type=int, default=0)
    ap.add_argument("--arena", type=float, default=0.0, help="GiB the process may allocate (0: the whole device)")
    ap.add_argument("--device-gb", type=float, default=180.0, help="device memory in GiB when --arena is not given")
    ap.add_argument("--context", type=int, default=0, help="longest sequence assumed for the workspace estimate")
    args = ap.parse_args(argv)
    cfg = _config(args)
    if not isinstance(cfg, GlmMoeDsaConfig):
        from ..utils.sizing import plan_dense
        p = plan_dense(cfg, world=args.world, batch_size=args.batch_size, chunk_size=args.chunk_size, max_pages=args.max_pages,
                       arena_gb=args.arena, device_gb=args.device_gb)
    else:
        p = plan_memory(cfg, world=args.world, cp=args.cp, ep=args.ep, mtp=args.mtp, batch_size=args.batch_size,
                        chunk_size=args.chunk_size, max_pages=args.max_pages, arena_gb=args.arena, device_gb=args.device_gb,
                        context=args.context)
    g = lambda b: f"{b / GIB:8.2f} GiB"       # noqa: E731
    print(f"replica of {args.world} GPU(s): tp={p.tp} cp={p.cp} ep={p.ep} mtp={args.mtp}   (per rank)")
    print(f"  weights                 {g(p.weights_bytes)}")
    print(f"  prefill workspace (est) {g(p.workspace_bytes)}   chunk {args.chunk_size}")
    print(f"  usable memory           {g(p.budget_bytes)}")
    print(f"  KV page                 {p.page_bytes / 1024:8.1f} KiB   = {p.tokens_per_page} tokens of one sequence")
    print(f"  pages that fit          {p.max_pages:8d}       = {p.max_tokens} tokens of context in total")
    verdict = "fit" if p.requested_fits else "DO NOT FIT"
    print(f"  pages asked for         {p.requested_pages:8d}       {verdict}  ({g(p.requested_pages * p.page_bytes).strip()})")
    print(json.dumps(p.to_dict()))
    return 0 if p.requested_fits else 1


if __name__ == "__main__":
    raise SystemExit(main())
