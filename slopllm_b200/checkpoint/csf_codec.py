"""NVFP4 compressed-scale codec `byte-window4-fixed-stream-u24-exceptions/1` (CPU, vectorised).

A logical E4M3 block-scale matrix [rows, columns] is stored as two planes:
  fixed       u8   per 16-row slab: 16 row-base bytes, then 16 x (columns/2) bytes of 4-bit
                   offsets (even column = low nibble, odd = high nibble)
  exceptions  u32  replacement words: low 24 bits = row-major position, top 8 bits = value,
                   strictly increasing positions
value(row, col) = exception if present else base[row] + nibble, with base <= 240 and values
<= 0x7e.  Padded TP shards use base 0x38 (E4M3 1.0) for appended rows and zero offsets for
appended columns.  Parity: `src/csf_codec.ts:1-366`.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np

SCHEMA = "lil-nvfp4-csf-checkpoint/1"
CODEC = "byte-window4-fixed-stream-u24-exceptions/1"
SUPPORTED_FAMILIES = ("glm53_744b_nvfp4",)
PADDED_SCALE_CODE = 0x38
MAX_SCALE_CODE = 0x7E
MAX_BASE = 240
FIXED_SUFFIX = ".nvfp4_csf_fixed"
EXC_SUFFIX = ".nvfp4_csf_exceptions"


class CsfContractError(ValueError):
    pass


def _geom(rows: int, columns: int) -> None:
    if rows <= 0 or columns <= 0 or rows % 16 or columns % 2:
        raise CsfContractError(f"NVFP4-CSF scale geometry [{rows}, {columns}] needs 16-row slabs and even columns")


def scale_geometry(weight_shape) -> Tuple[int, int]:
    """Logical scale geometry of a packed NVFP4 weight [N, K/2]: [N, K/16]."""
    if len(weight_shape) != 2 or weight_shape[0] <= 0 or weight_shape[1] <= 0 or weight_shape[1] % 8:
        raise CsfContractError(f"NVFP4 weight shape {list(weight_shape)} is not a valid [N, K/2] nibble pack")
    return weight_shape[0], weight_shape[1] // 8


def fixed_stream_length(rows: int, columns: int) -> int:
    _geom(rows, columns)
    return (rows // 16) * 16 * (1 + columns // 2)


def _split_fixed(fixed: np.ndarray, rows: int, columns: int):
    """-> (bases [rows], packed [rows, columns/2]) views of the fixed stream."""
    sel = columns // 2
    slabs = fixed.reshape(rows // 16, 16 * (1 + sel))
    bases = slabs[:, :16].reshape(rows)
    packed = slabs[:, 16:].reshape(rows, sel)
    return bases, packed


def validate_fixed_plane(fixed: np.ndarray, rows: int, columns: int) -> None:
    _geom(rows, columns)
    want = fixed_stream_length(rows, columns)
    if fixed.size != want:
        raise CsfContractError(f"NVFP4-CSF fixed stream must be {want} bytes for a {rows}x{columns} scale matrix, got {fixed.size}")
    bases, _ = _split_fixed(fixed, rows, columns)
    if bases.size and int(bases.max()) > MAX_BASE:
        raise CsfContractError(f"NVFP4-CSF row base {int(bases.max())} exceeds the 0..{MAX_BASE} window")


def decode_exceptions(exceptions: np.ndarray, rows: int, columns: int):
    raw = np.ascontiguousarray(exceptions).view(np.uint8)
    if raw.size % 4:
        raise CsfContractError(f"NVFP4-CSF exception plane must be whole uint32 words, got {raw.size} bytes")
    words = raw.view("<u4")
    pos = (words & 0xFFFFFF).astype(np.int64)
    val = (words >> 24).astype(np.uint8)
    if pos.size:
        if int(pos.max()) >= rows * columns:
            raise CsfContractError(f"NVFP4-CSF exception position {int(pos.max())} is outside the {rows}x{columns} scale matrix")
        if np.any(np.diff(pos) <= 0):
            raise CsfContractError("NVFP4-CSF exception positions must be sorted and unique")
    return pos, val


def _reject_invalid(values: np.ndarray, what: str) -> None:
    if values.size and int(values.max()) > MAX_SCALE_CODE:
        raise CsfContractError(f"NVFP4-CSF {what} contains invalid E4M3 scale code 0x{int(values.max()):x}")


def expand_scale_planes(fixed, exceptions, rows: int, columns: int) -> np.ndarray:
    """Lossless expansion into row-major E4M3 scale bytes [rows, columns] (all contract checks)."""
    fixed = np.frombuffer(fixed, dtype=np.uint8) if not isinstance(fixed, np.ndarray) else fixed.reshape(-1)
    validate_fixed_plane(fixed, rows, columns)
    pos, val = decode_exceptions(np.asarray(exceptions), rows, columns)
    bases, packed = _split_fixed(fixed, rows, columns)
    out = np.empty((rows, columns), dtype=np.uint16)
    out[:, 0::2] = bases[:, None].astype(np.uint16) + (packed & 0x0F)
    out[:, 1::2] = bases[:, None].astype(np.uint16) + (packed >> 4)
    out = out.astype(np.uint8)
    flat = out.reshape(-1)
    flat[pos] = val
    _reject_invalid(flat, "scale values")
    return out


def expand_scale_window(fixed, exceptions, rows, columns, row0, row_len, col0, col_len) -> np.ndarray:
    """Expansion of the window [row0:row0+row_len, col0:col0+col_len]; plane invariants are still
    validated over the whole plane."""
    if min(row0, row_len, col0, col_len) < 0 or row0 + row_len > rows or col0 + col_len > columns:
        raise CsfContractError(f"NVFP4-CSF window [{row0}+{row_len}, {col0}+{col_len}] is outside the {rows}x{columns} scale matrix")
    full = expand_scale_planes(fixed, exceptions, rows, columns)
    return np.ascontiguousarray(full[row0:row0 + row_len, col0:col0 + col_len])


def compress_scales(scales: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Encoder: [rows, columns] u8 scale codes -> (fixed u8, exceptions u32).  Row base = the
    minimum of the row clamped to 240; values more than 15 above the base become exceptions."""
    s = np.ascontiguousarray(scales, dtype=np.uint8)
    rows, columns = s.shape
    _geom(rows, columns)
    _reject_invalid(s, "source scales")
    bases = np.minimum(s.min(axis=1), MAX_BASE).astype(np.uint8)
    off = s.astype(np.int16) - bases[:, None]
    exc_mask = off > 15
    nib = np.where(exc_mask, 0, off).astype(np.uint8)
    packed = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    sel = columns // 2
    fixed = np.empty((rows // 16, 16 * (1 + sel)), dtype=np.uint8)
    fixed[:, :16] = bases.reshape(rows // 16, 16)
    fixed[:, 16:] = packed.reshape(rows // 16, 16 * sel)
    pos = np.flatnonzero(exc_mask.reshape(-1)).astype(np.uint32)
    if pos.size and int(pos.max()) >= 1 << 24:
        raise CsfContractError("scale matrix too large for 24-bit exception positions")
    words = (s.reshape(-1)[pos].astype(np.uint32) << 24) | pos
    return fixed.reshape(-1), words.astype("<u4")


def slice_scale_planes(fixed, exceptions, rows, columns, row_slice, col_slice, out_rows: Optional[int] = None,
                       out_columns: Optional[int] = None):
    """Slice compressed planes to a TP shard without decoding to bytes, rebasing exception
    positions; `out_rows` / `out_columns` pad the shard (base 0x38 rows, zero offset columns)."""
    fixed = np.frombuffer(fixed, dtype=np.uint8) if not isinstance(fixed, np.ndarray) else fixed.reshape(-1)
    validate_fixed_plane(fixed, rows, columns)
    pos, val = decode_exceptions(np.asarray(exceptions), rows, columns)
    r0, r1 = row_slice
    c0, c1 = col_slice
    if not (0 <= r0 < r1 <= rows and r0 % 16 == 0 and r1 % 16 == 0):
        raise CsfContractError("NVFP4-CSF row slices require complete 16-row slabs")
    if not (0 <= c0 < c1 <= columns and c0 % 2 == 0 and c1 % 2 == 0):
        raise CsfContractError("NVFP4-CSF column slices require complete nibble pairs")
    sr, sc = r1 - r0, c1 - c0
    orows = sr if out_rows is None else out_rows
    ocols = sc if out_columns is None else out_columns
    if not (orows >= sr and orows % 16 == 0 and ocols >= sc and ocols % 2 == 0):
        raise CsfContractError("NVFP4-CSF padded slices must extend whole slabs and pairs")
    bases, packed = _split_fixed(fixed, rows, columns)
    ob = np.full(orows, PADDED_SCALE_CODE, dtype=np.uint8)
    op = np.zeros((orows, ocols // 2), dtype=np.uint8)
    ob[:sr] = bases[r0:r1]
    op[:sr, : sc // 2] = packed[r0:r1, c0 // 2:c1 // 2]
    out_fixed = np.empty((orows // 16, 16 * (1 + ocols // 2)), dtype=np.uint8)
    out_fixed[:, :16] = ob.reshape(orows // 16, 16)
    out_fixed[:, 16:] = op.reshape(orows // 16, 16 * (ocols // 2))
    prow, pcol = pos // columns, pos % columns
    keep = (prow >= r0) & (prow < r1) & (pcol >= c0) & (pcol < c1)
    npos = ((prow[keep] - r0) * ocols + (pcol[keep] - c0)).astype(np.uint32)
    words = (val[keep].astype(np.uint32) << 24) | npos
    return out_fixed.reshape(-1), words.astype("<u4")


def concat_fc1_scale_planes(first, second, local_rows: int, columns: int):
    """Fuse two projections' planes along rows (gate/up -> W13); the second one's exception
    positions shift by local_rows * columns."""
    f1, e1 = first
    f2, e2 = second
    want = fixed_stream_length(local_rows, columns)
    if f1.size != want or f2.size != want:
        raise CsfContractError("NVFP4-CSF FC1 fusion requires equal fixed-stream geometry for both projections")
    shift = local_rows * columns
    w2 = np.asarray(e2).view("<u4")
    p2 = (w2 & 0xFFFFFF) + shift
    if p2.size and int(p2.max()) >= 2 * shift:
        raise CsfContractError("NVFP4-CSF fused exception position is outside the fused matrix")
    fused = np.concatenate([np.asarray(e1).view("<u4"), ((w2 >> 24) << 24) | p2.astype(np.uint32)]).astype("<u4")
    decode_exceptions(fused, 2 * local_rows, columns)
    return np.concatenate([f1, f2]), fused


def tp_extent(intermediate: int, tp_rank: int, tp_size: int, alignment: int) -> Tuple[int, int]:
    if tp_size <= 0 or not (0 <= tp_rank < tp_size) or intermediate <= 0 or intermediate % (alignment * tp_size):
        raise CsfContractError(f"CSF requires a valid TP rank and extents aligned to {alignment} intermediate channels")
    local = intermediate // tp_size
    return tp_rank * local, (tp_rank + 1) * local
