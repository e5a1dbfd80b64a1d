"""GPU expansion of CSF scale planes (the loader's fast path; `csrc/csf.cu`)."""
from __future__ import annotations

import numpy as np
import torch

from ..ops import native as N
from .csf_codec import CsfContractError, fixed_stream_length

_status = {}


def _status_word(device) -> torch.Tensor:
    key = torch.device(device).index or 0
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def decode_csf_scales(fixed: np.ndarray, exceptions: np.ndarray, rows: int, cols: int, row0: int, out_rows: int, col0: int,
                      out_cols: int, device) -> torch.Tensor:
    """Upload the two planes and decode the window on the device.  Returns float8_e4m3fn
    [out_rows, out_cols].  Violations are recorded in a per-device status word that
    `check_decode_status` turns into a `CsfContractError` at the end of the load."""
    if fixed.size != fixed_stream_length(rows, cols):
        raise CsfContractError(f"NVFP4-CSF fixed stream has {fixed.size} bytes, geometry {rows}x{cols} needs "
                               f"{fixed_stream_length(rows, cols)}")
    N._SIGS.setdefault("sl_csf_decode", [N.vp, N.vp, N.vp, N.i32, N.i32, N.i32, N.i32, N.i32, N.i32, N.i32, N.vp, N.vp])
    f = torch.from_numpy(np.ascontiguousarray(fixed).copy()).to(device, non_blocking=True)
    e = torch.from_numpy(np.ascontiguousarray(exceptions).view(np.int32).copy()).to(device, non_blocking=True)
    out = torch.empty(out_rows, out_cols, dtype=torch.uint8, device=device)
    N.call("sl_csf_decode", out.data_ptr(), f.data_ptr(), e.data_ptr() if e.numel() else 0, int(e.numel()), rows, cols, row0,
           out_rows, col0, out_cols, _status_word(device).data_ptr(), N.stream())
    return out.view(torch.float8_e4m3fn)


def check_decode_status(device) -> None:
    code = int(_status_word(device).item())
    if code:
        _status_word(device).zero_()
        what = [m for bit, m in ((1, "scale code above 0x7e"), (2, "exception words unsorted or out of range"),
                                 (4, "row base above 240")) if code & bit]
        raise CsfContractError("CSF GPU decode reported: " + ", ".join(what))
