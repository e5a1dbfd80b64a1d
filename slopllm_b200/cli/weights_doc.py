"""Write a Markdown inventory of a checkpoint's tensors, grouped by name pattern.

    python -m slopllm_b200 weights-doc --model <dir|hub id> [--output weights.md]

Layer indices become `N` (`MTP` for layers past `num_hidden_layers`) and expert indices `E`, so the table has one
row per (pattern, shape, dtype) with its count and total size.  Works on plain safetensors shards and on CSF
containers (through `checkpoint.source`).  Reference: `scripts/gen_glm51_weights_md.py`, which produces
`GLM51-NVFP4-weights.md`.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
from collections import defaultdict
from typing import Dict, Iterable, List, Tuple

DTYPE_SIZES = {"BOOL": 1, "U8": 1, "I8": 1, "F8_E4M3": 1, "F8_E5M2": 1, "I16": 2, "U16": 2, "F16": 2, "BF16": 2,
               "I32": 4, "U32": 4, "F32": 4, "I64": 8, "U64": 8, "F64": 8}


def human(n: int) -> str:
    for unit, size in (("GB", 1 << 30), ("MB", 1 << 20), ("KB", 1 << 10)):
        if n >= size:
            return f"{n / size:.2f} {unit}"
    return f"{n} B"


def pattern_of(name: str, num_layers: int | None) -> Tuple[str, bool]:
    """(pattern, is_mtp): `model.layers.12.mlp.experts.7.x` -> `model.layers.N.mlp.experts.E.x`."""
    mtp = False

    def layer(m):
        nonlocal mtp
        if num_layers is not None and int(m.group(1)) >= num_layers:
            mtp = True
            return "layers.MTP."
        return "layers.N."
    p = re.sub(r"layers\.(\d+)\.", layer, name)
    p = re.sub(r"experts\.(\d+)\.", "experts.E.", p)
    return p, mtp


def inventory(metas: Iterable[Tuple[str, str, Tuple[int, ...]]], num_layers: int | None) -> List[Dict]:
    groups: Dict[Tuple[str, Tuple[int, ...], str, bool], List[int]] = defaultdict(lambda: [0, 0])
    for name, dtype, shape in metas:
        n = DTYPE_SIZES.get(dtype, 0)
        for d in shape:
            n *= d
        pat, mtp = pattern_of(name, num_layers)
        g = groups[(pat, tuple(shape), dtype, mtp)]
        g[0] += 1
        g[1] += n
    rows = [{"pattern": k[0], "shape": list(k[1]), "dtype": k[2], "mtp": k[3], "count": v[0], "bytes": v[1]} for k, v in groups.items()]
    rows.sort(key=lambda r: (r["pattern"], r["shape"], r["dtype"]))
    return rows


def render(rows: List[Dict], source: str, cfg: Dict) -> str:
    total_n = sum(r["count"] for r in rows)
    total_b = sum(r["bytes"] for r in rows)
    out = ["# Weight inventory", "", f"Source: `{source}`", "", "## Overview", "",
           f"- **Total tensors**: {total_n:,}", f"- **Total size**: {total_b:,} bytes ({human(total_b)})"]
    if cfg:
        for k in ("model_type", "num_hidden_layers", "first_k_dense_replace", "n_routed_experts", "num_nextn_predict_layers"):
            if k in cfg:
                out.append(f"- **{k}**: {cfg[k]}")
    out += ["", "## Tensor name patterns", "", "`N` = layer index, `E` = expert index, `MTP` = a layer past `num_hidden_layers`.", "",
            "| Pattern | Shape | Dtype | Count | Total size |", "|---|---|---|---|---|"]
    for r in rows:
        out.append(f"| `{r['pattern']}`{' **MTP**' if r['mtp'] else ''} | {r['shape']} | {r['dtype']} | {r['count']} | {human(r['bytes'])} |")
    return "\n".join(out) + "\n"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="slopllm_b200.cli.weights_doc")
    ap.add_argument("--model", required=True)
    ap.add_argument("--output", default=None, help="Markdown file to write (default: standard output)")
    args = ap.parse_args(argv)
    from ..checkpoint.source import open_checkpoint_source
    from ..utils.model_path import resolve_model_path
    path = resolve_model_path(args.model)
    src = open_checkpoint_source(path)
    cfg = {}
    cfg_path = os.path.join(src.config_dir, "config.json")
    if os.path.exists(cfg_path):
        with open(cfg_path) as f:
            cfg = json.load(f)
    metas = []
    for name in src.names():
        dtype, shape = src.meta(name)
        metas.append((name, dtype, tuple(shape)))
    src.close()
    text = render(inventory(metas, cfg.get("num_hidden_layers")), args.model, cfg)
    if args.output:
        with open(args.output, "w") as f:
            f.write(text)
    else:
        sys.stdout.write(text)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
