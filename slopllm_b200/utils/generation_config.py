"""Sampling defaults that ship with a checkpoint.

`generation_config.json` (and, below it, `config.json`) may carry `temperature`, `top_p`, `top_k`, `repetition_penalty`
and `max_new_tokens`.  The server uses them for every flag the operator did not give on the command line, before its
own built-in defaults.  Reference: `loadGenerationConfig`, `loadMaxPositionEmbeddings` (`src/chat_model.ts:127-150`) and
their use in `src/openai-server.ts:424-435`.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

_KEYS = {"temperature": float, "top_p": float, "top_k": int, "repetition_penalty": float, "max_new_tokens": int}


def _read(path: str) -> dict:
    try:
        with open(path) as f:
            d = json.load(f)
        return d if isinstance(d, dict) else {}
    except (OSError, ValueError):
        return {}


def load_generation_defaults(model_dir: Optional[str]) -> Dict[str, float]:
    """{key: value} for the keys above that the checkpoint defines as numbers; `generation_config.json` wins over
    `config.json`.  Booleans and strings are ignored (some checkpoints carry `"temperature": null`)."""
    if not model_dir:
        return {}
    raw = {**_read(os.path.join(model_dir, "config.json")), **_read(os.path.join(model_dir, "generation_config.json"))}
    out: Dict[str, float] = {}
    for k, cast in _KEYS.items():
        v = raw.get(k)
        if isinstance(v, (int, float)) and not isinstance(v, bool):
            out[k] = cast(v)
    return out


def max_position_embeddings(model_dir: Optional[str]) -> Optional[int]:
    """The context length the checkpoint was trained for (`text_config` of multimodal configs first)."""
    if not model_dir:
        return None
    raw = _read(os.path.join(model_dir, "config.json"))
    cfg = raw.get("text_config") if isinstance(raw.get("text_config"), dict) else raw
    v = cfg.get("max_position_embeddings")
    return int(v) if isinstance(v, int) and not isinstance(v, bool) else None


def apply_generation_defaults(args, model_dir: Optional[str], builtin: Dict[str, float]) -> Dict[str, str]:
    """Fill every sampling attribute of `args` that is still None: checkpoint value first, then `builtin`.
    Returns where each value came from ("flag" / "checkpoint" / "default"), for the start-up log."""
    ckpt = load_generation_defaults(model_dir)
    names = {"temperature": "temperature", "top_p": "top_p", "top_k": "top_k", "repetition_penalty": "repetition_penalty",
             "max_tokens": "max_new_tokens"}
    origin = {}
    for attr, key in names.items():
        if getattr(args, attr, None) is not None:
            origin[attr] = "flag"
        elif key in ckpt:
            setattr(args, attr, ckpt[key])
            origin[attr] = "checkpoint"
        else:
            setattr(args, attr, builtin[attr])
            origin[attr] = "default"
    return origin
