"""Uniform view over a checkpoint directory: plain safetensors shards or a CSF container.

Parity: `src/checkpoint_source.ts:1-336` — consumers iterate logical tensors and never see
the physical planes, except through `csf_planes()` which hands the compressed planes to the
GPU decoder.
"""
from __future__ import annotations

import os
from typing import Dict, Iterator, List, Optional, Tuple

import numpy as np
import torch

from .csf_container import CsfContainer, looks_like_csf
from .safetensors_io import SafetensorsFile, iter_dir


class CheckpointSource:
    def __init__(self, model_dir: str):
        self.dir = model_dir
        self.csf: Optional[CsfContainer] = CsfContainer(model_dir) if looks_like_csf(model_dir) else None
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        if self.csf is None:
            for path in iter_dir(model_dir):
                st = SafetensorsFile(path)
                self._files[path] = st
                for n in st.names():
                    self._where[n] = path

    @property
    def config_dir(self) -> str:
        return os.path.join(self.dir, "metadata") if self.csf is not None else self.dir

    def names(self) -> List[str]:
        return self.csf.names() if self.csf is not None else list(self._where)

    def has(self, name: str) -> bool:
        return name in (self.csf.source_names if self.csf is not None else self._where)

    def meta(self, name: str) -> Tuple[str, Tuple[int, ...]]:
        if self.csf is not None:
            return self.csf.meta(name)
        m = self._files[self._where[name]].meta(name)
        return m.dtype, m.shape

    def tensor(self, name: str) -> torch.Tensor:
        if self.csf is not None:
            return self.csf.tensor(name)
        return self._files[self._where[name]].tensor(name)

    def window(self, name: str, rows=None, cols=None, pin: bool = False) -> Optional[torch.Tensor]:
        """Contiguous host copy of a row / column window of a tensor stored in a plain safetensors shard, made by the C++
        runtime (`SafetensorsFile.window`); None when the tensor lives in a CSF container or the runtime is not built."""
        if self.csf is not None or name not in self._where:
            return None
        return self._files[self._where[name]].window(name, rows, cols, pin=pin)

    def csf_planes(self, name: str) -> Optional[Tuple[np.ndarray, np.ndarray, Tuple[int, int]]]:
        """(fixed, exceptions, (rows, columns)) of a replaced scale tensor, else None."""
        if self.csf is None or not self.csf.is_compressed(name):
            return None
        fixed, exc = self.csf.planes(name)
        return fixed, exc, self.csf.scales[name].shape

    def __iter__(self) -> Iterator[str]:
        return iter(self.names())

    def close(self) -> None:
        if self.csf is not None:
            self.csf.close()
        for st in self._files.values():
            st.close()


def open_checkpoint_source(model_dir: str) -> CheckpointSource:
    return CheckpointSource(model_dir)
