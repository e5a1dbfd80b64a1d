"""safetensors reader / writer (header JSON + memory-mapped tensor ranges).

Parity: `src/safetensors.ts:1-166`.  The reader never copies: tensors are views on one
`mmap` of the file, so a TP rank can take a strided window of a tensor and upload only that.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import threading
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "U32": (torch.uint32, 4), "U16": (torch.uint16, 2), "BOOL": (torch.bool, 1), "F8_E4M3": (torch.float8_e4m3fn, 1),
    "F8_E5M2": (torch.float8_e5m2, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass
class TensorMeta:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int            # byte offsets relative to the data section
    end: int

    @property
    def nbytes(self) -> int:
        return self.end - self.begin

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype][0]


class SafetensorsFile:
    PIN_MIN_BYTES = 256 << 10

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise ValueError(f"{path}: not a safetensors file")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8 or n > 1 << 30:
            raise ValueError(f"{path}: bad header length {n}")
        self.header_bytes = self._f.read(n)
        header = json.loads(self.header_bytes)
        self.metadata: Dict[str, str] = header.pop("__metadata__", {}) or {}
        self.data_offset = 8 + n
        self.file_size = size
        self.tensors: Dict[str, TensorMeta] = {}
        for name, t in header.items():
            b, e = t["data_offsets"]
            if t["dtype"] not in _DTYPES:
                raise ValueError(f"{path}: tensor {name} has unsupported dtype {t['dtype']}")
            meta = TensorMeta(name, t["dtype"], tuple(t["shape"]), b, e)
            want = int(np.prod(meta.shape, dtype=np.int64)) * _DTYPES[meta.dtype][1] if meta.shape else _DTYPES[meta.dtype][1]
            if e - b != want or e > size - self.data_offset:
                raise ValueError(f"{path}: tensor {name} extent {e - b} does not match its shape/dtype ({want} bytes)")
            self.tensors[name] = meta
        self._mm: Optional[mmap.mmap] = None
        self._native = None               # C++ mapping of the same file, opened on the first window() call
        self._native_lock = threading.Lock()

    def _map(self) -> mmap.mmap:
        if self._mm is None:
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        return self._mm

    def names(self) -> List[str]:
        return list(self.tensors)

    def meta(self, name: str) -> TensorMeta:
        return self.tensors[name]

    def tensor_offset(self, name: str) -> int:
        """Absolute file offset of the tensor's first byte."""
        return self.data_offset + self.tensors[name].begin

    def read_bytes(self, name: str) -> memoryview:
        m = self.tensors[name]
        return memoryview(self._map())[self.data_offset + m.begin:self.data_offset + m.end]

    def tensor(self, name: str) -> torch.Tensor:
        """Zero-copy CPU tensor backed by the mapping (do not write to it)."""
        m = self.tensors[name]
        dt, _ = _DTYPES[m.dtype]
        if m.nbytes == 0:
            return torch.empty(m.shape, dtype=dt)
        raw = np.frombuffer(self._map(), dtype=np.uint8, count=m.nbytes, offset=self.data_offset + m.begin)
        t = torch.from_numpy(raw)
        return t.view(dt).reshape(m.shape) if dt != torch.uint8 else t.reshape(m.shape)

    def window(self, name: str, rows: Optional[Tuple[int, int]] = None, cols: Optional[Tuple[int, int]] = None,
               pin: bool = False, threads: int = 4) -> Optional[torch.Tensor]:
        """Contiguous copy of rows [r0, r1) x columns [c0, c1) of a 2-D tensor (1-D: rows only), made by the C++
        runtime's strided multi-threaded copy straight out of the mapping into a fresh (optionally pinned) host tensor.
        This is what a tensor-parallel rank uploads.  Returns None when the native runtime is not built or the tensor
        has another rank; callers then slice `tensor()`."""
        m = self.tensors[name]
        if len(m.shape) not in (1, 2) or m.nbytes == 0:
            return None
        try:
            from ..runtime.native_runtime import MappedFile
            with self._native_lock:                       # loader threads share the file object
                if self._native is None:
                    self._native = MappedFile(self.path)
        except Exception:  # noqa: BLE001  (library not built: the Python mapping serves the read)
            return None
        dt, esz = _DTYPES[m.dtype]
        R = m.shape[0]
        Cn = m.shape[1] if len(m.shape) == 2 else 1
        r0, r1 = rows or (0, R)
        c0, c1 = cols or (0, Cn)
        if not (0 <= r0 <= r1 <= R and 0 <= c0 <= c1 <= Cn) or (len(m.shape) == 1 and cols is not None):
            raise IndexError(f"{name}: window rows {rows} cols {cols} outside shape {m.shape}")
        shape = (r1 - r0, c1 - c0) if len(m.shape) == 2 else (r1 - r0,)
        nbytes = (r1 - r0) * (c1 - c0) * esz
        # small windows (norm weights, per-expert scales) are not worth a pinned block
        out = torch.empty(shape, dtype=dt, pin_memory=pin and nbytes >= self.PIN_MIN_BYTES and torch.cuda.is_available())
        if out.numel():
            self._native.copy_rows(self.data_offset + m.begin + (r0 * Cn + c0) * esz, Cn * esz, (c1 - c0) * esz, r1 - r0,
                                   out.data_ptr(), threads)
        return out

    def close(self) -> None:
        if self._native is not None:
            self._native.close()
            self._native = None
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass                      # tensors still reference the mapping: the GC closes it later
            self._mm = None
        self._f.close()


def _as_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous().reshape(-1)
    return t.view(torch.uint8).numpy().tobytes() if t.numel() else b""


def serialize(tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> bytes:
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    off = 0
    blobs: List[bytes] = []
    for name, t in tensors.items():
        b = _as_bytes(t)
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        off += len(b)
        blobs.append(b)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    return struct.pack("<Q", len(hj)) + hj + b"".join(blobs)


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> int:
    data = serialize(tensors, metadata)
    with open(path, "wb") as f:
        f.write(data)
    return len(data)


def iter_dir(model_dir: str) -> Iterable[str]:
    """Shard files of a checkpoint directory in index order (or sorted *.safetensors)."""
    idx = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            wm = json.load(f)["weight_map"]
        seen: List[str] = []
        for fn in wm.values():
            if fn not in seen:
                seen.append(fn)
        return [os.path.join(model_dir, s) for s in seen]
    return sorted(os.path.join(model_dir, f) for f in os.listdir(model_dir) if f.endswith(".safetensors"))
