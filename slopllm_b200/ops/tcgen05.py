"""Python entry points of the tcgen05 (TMEM / TMA) GEMM kernels."""
from __future__ import annotations

import torch

from . import native as N

_err = {}
_reset_hooks = {}

ERROR_WORDS = 16        # [0] tcgen05 expired wait, [4..7] index self-check, [8..11] persistent-kernel wait, [12..15] collective wait


def error_flag(device) -> torch.Tensor:
    """Per-device block of int32 status words that kernels write when a bounded wait expires or an index self-check
    fails: one place, so that the engine reads everything back with the step's result in a single copy."""
    key = torch.device(device).index or 0
    if key not in _err:
        _err[key] = torch.zeros(ERROR_WORDS, dtype=torch.int32, device=device)
    return _err[key]


def on_error_reset(device, hook) -> None:
    """`hook()` runs when an error of this device is reported (kernels that gave up leave their counters as they were)."""
    _reset_hooks.setdefault(torch.device(device).index or 0, []).append(hook)


def raise_for(words, device) -> None:
    """Turn a host copy of the status block into an exception (and clear the device block)."""
    if not any(words[i] for i in (0, 4, 8, 12)):
        return
    error_flag(device).zero_()
    for hook in _reset_hooks.get(torch.device(device).index or 0, []):
        hook()
    if words[12]:
        raise N.CollectiveTimeout(f"device wait on a peer expired at site {words[13]} (expected flag {words[14]}, saw {words[15]})")
    if words[8]:
        raise N.NativeError(f"persistent kernel wait expired at site {words[9]} (expected {words[10]}, saw {words[11]})")
    if words[0]:
        raise N.NativeError(f"tcgen05 kernel reported an expired wait (site {words[0]})")
    raise N.NativeError(f"index self-check failed at site {words[4]}: value {words[5]} outside [0, {words[6]}) in block {words[7]}")


def check_errors(device) -> None:
    raise_for(error_flag(device).tolist(), device)


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out_f32: bool = False, bn: int = 0) -> torch.Tensor:
    """y[M, N] = x[M, K] @ w[N, K]^T on tcgen05 tensor cores (bf16 in, fp32 accumulate).
    `bn` is the tile width (64 / 128 / 256); 0 picks 128 x 256 tiles when the output is at least 512 columns wide
    (measured 1.25 - 1.45 times faster than 128 x 128 at 4096 rows)."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    if x.stride(-1) != 1:
        x = x.contiguous()
    if w.stride(-1) != 1:
        w = w.contiguous()
    M, K = x.shape
    Nn = w.shape[0]
    if bn == 0:
        bn = 256 if Nn >= 512 else 128
        row_tiles = (M + 127) // 128
        while bn > 64 and row_tiles * ((Nn + bn - 1) // bn) < 148:       # fewer tiles than SMs: narrower tiles (router: 256 columns)
            bn //= 2
    pad = 4 if out_f32 else 8                        # 16-byte aligned rows for the vector stores
    ld = (Nn + pad - 1) // pad * pad
    y = torch.empty(M, ld, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)[:, :Nn]
    N.call("sl_gemm_bf16_tcgen05", x.data_ptr(), w.data_ptr(), y.data_ptr(), M, Nn, K, x.stride(0), w.stride(0),
           y.stride(0), int(out_f32), error_flag(x.device).data_ptr(), bn, N.stream())
    return y
