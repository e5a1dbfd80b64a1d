"""`model_type` -> loader and capabilities.  Reference: `src/model_registry.ts:1-56`."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, Optional

import torch

from ..parallel.dist import ParallelContext


@dataclass
class ModelRegistration:
    phased_prefill: bool
    context_parallel: bool
    mtp: bool
    persistent_loader: bool
    load: Callable            # (model_dir, ctx, mtp) -> (cfg, model)


def _load_glm_moe_dsa(model_dir: str, ctx: ParallelContext, mtp: int = 0):
    from ..checkpoint.loader import load_model
    from ..parallel.fused import make_comm
    from .glm_moe_dsa import GlmMoeDsaModel
    dtype = torch.bfloat16 if ctx.device.type == "cuda" else torch.float32
    tp_world = ctx.world          # weights stay tensor-parallel under context parallelism too
    cfg, w = load_model(model_dir, ctx.device, dtype, ctx.rank if tp_world > 1 else 0, tp_world, ep=ctx.ep, with_mtp=mtp > 0)
    return cfg, GlmMoeDsaModel(cfg, w, ctx, comm=make_comm(ctx, cfg))


def _load_dense(model_dir: str, ctx: ParallelContext, mtp: int = 0):
    from .dense import load_dense_model
    return load_dense_model(model_dir, ctx)


def _load_glm5_next(model_dir: str, ctx: ParallelContext, mtp: int = 0):
    from .glm5_next import Glm5NextModel
    m = Glm5NextModel.from_pretrained(model_dir, ctx)
    return m.cfg, m


MODEL_REGISTRY: Dict[str, ModelRegistration] = {
    "glm_moe_dsa": ModelRegistration(True, True, True, True, _load_glm_moe_dsa),
    "glm5_next": ModelRegistration(False, False, False, True, _load_glm5_next),
    "qwen3": ModelRegistration(False, False, False, True, _load_dense),
    "qwen3_5": ModelRegistration(False, False, False, False, _load_dense),
}


def checkpoint_config_dir(model_dir: str) -> str:
    """A CSF container keeps the model's config under `metadata/`."""
    if not os.path.isfile(os.path.join(model_dir, "config.json")) and os.path.isfile(os.path.join(model_dir, "metadata", "config.json")):
        return os.path.join(model_dir, "metadata")
    return model_dir


def inspect_model(model_dir: str, cp: bool = False, mtp: int = 0):
    """(model_type, registration, raw config) with the option checks of the reference's `inspectModel`."""
    path = os.path.join(checkpoint_config_dir(model_dir), "config.json")
    with open(path) as f:
        config = json.load(f)
    mt = config.get("model_type")
    if not isinstance(mt, str) or mt not in MODEL_REGISTRY:
        raise ValueError(f"unsupported model_type {mt!r} in {path}; supported types: {', '.join(MODEL_REGISTRY)}")
    reg = MODEL_REGISTRY[mt]
    if cp and not reg.context_parallel:
        raise ValueError(f"{mt} does not support --cp")
    if mtp > 0 and not reg.mtp:
        raise ValueError(f"{mt} does not support --mtp")
    return mt, reg, config


def load_any(model_dir: str, ctx: Optional[ParallelContext] = None, mtp: int = 0):
    ctx = ctx or ParallelContext()
    _, reg, _ = inspect_model(model_dir, cp=ctx.cp, mtp=mtp)
    return reg.load(model_dir, ctx, mtp)
