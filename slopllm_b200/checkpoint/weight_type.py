"""Map a checkpoint tensor (dtype + name + neighbours) to the internal weight type.

Parity: `src/weight_type.ts:1-80` — a `U8` weight whose sibling `weight_scale` exists is a
packed 4-bit weight: NVFP4 when the scale is E4M3 (block of 16), MXFP4 when it is an 8-bit
exponent (block of 32); an F8_E4M3 weight with `weight_scale_inv` is block-quantised FP8.
"""
from __future__ import annotations

from typing import Callable, Optional


def resolve_weight_type(name: str, dtype: str, scale_dtype_of: Callable[[str], Optional[str]]) -> str:
    if not name.endswith(".weight"):
        return dtype
    base = name[: -len(".weight")]
    if dtype == "U8":
        sd = scale_dtype_of(base + ".weight_scale")
        if sd == "F8_E4M3":
            return "U8_NVFP4"
        if sd in ("U8", "F8_E8M0"):
            return "U8_MXFP4"
        return "U8"
    if dtype == "F8_E4M3":
        if scale_dtype_of(base + ".weight_scale_inv") is not None:
            return "F8_E4M3_BLOCK"
        return "F8_E4M3"
    return dtype


def is_quant_aux(name: str) -> bool:
    """Auxiliary tensors of a quantised linear (consumed with the weight, not loaded alone)."""
    return name.endswith((".weight_scale", ".weight_scale_2", ".input_scale", ".weight_scale_inv"))
