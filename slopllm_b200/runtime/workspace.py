"""Arena workspace with stream lineage, and small lifetime helpers.

PyTorch's caching allocator serves the engine's transient tensors; this module is for callers that
need the reference's explicit model: one device arena (weights, caches and step buffers carved
from a single allocation that can be exported over CUDA IPC), buffers that may only be reused on
the stream that freed them, scopes that release everything allocated inside, and `freeze()` for
long-lived allocations.  Offsets come from the native first-fit heap (`csrc/runtime/page_pool.cpp`).

Reference: `src/workspace.ts:1-323` (WorkspaceBase), `src/heap.ts:1-209`, `src/using-holder.ts:1-63`,
`src/tensor-tree.ts:1-29`.
"""
from __future__ import annotations

from contextlib import contextmanager
from dataclasses import dataclass
from typing import Any, Callable, Dict, Generic, Iterator, List, Optional, Tuple, TypeVar

import torch

from .native_runtime import Heap

T = TypeVar("T")


@dataclass
class _Block:
    offset: int
    nbytes: int
    stream: int                      # lineage: stream on which the block was last used / freed
    name: str = ""


class Workspace:
    """Sub-allocates tensors from one backing buffer.

    * `alloc(shape, dtype)` returns a view into the arena; `free(tensor)` gives the range back.
    * A block freed on stream s goes to s's own free list and is reused first by allocations on s
      (no synchronisation needed); another stream may take it only after `promote(s)` (the caller
      has made that stream wait for s, e.g. with an event).
    * `scope()` frees everything allocated inside on exit; `freeze()` marks current allocations as
      permanent (they survive scopes and `reset`).
    """

    def __init__(self, nbytes: int, device="cpu", alignment: int = 256, pinned: bool = False):
        self.device = torch.device(device)
        self.nbytes = nbytes
        raw = torch.empty(nbytes + alignment, dtype=torch.uint8, device=self.device,
                          pin_memory=pinned and self.device.type == "cpu" and torch.cuda.is_available())
        pad = (-raw.data_ptr()) % alignment                # host allocations are not aligned to 256 bytes by themselves
        self._raw = raw
        self.buffer = raw[pad:pad + nbytes]
        self.heap = Heap(nbytes, alignment)
        self.live: Dict[int, _Block] = {}                 # data_ptr -> block
        self.free_by_stream: Dict[int, List[_Block]] = {}
        self.frozen: set = set()
        self._scopes: List[List[int]] = []
        self.peak = 0

    # -- allocation ------------------------------------------------------------------------------------------
    def _take_lineage(self, nbytes: int, stream: int) -> Optional[_Block]:
        lst = self.free_by_stream.get(stream, [])
        for i, b in enumerate(lst):
            if b.nbytes >= nbytes:
                return lst.pop(i)
        return None

    def alloc(self, shape, dtype=torch.bfloat16, name: str = "", stream: int = 0) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = max(1, n * torch.empty((), dtype=dtype).element_size())
        blk = self._take_lineage(nbytes, stream)
        if blk is None:
            off = self.heap.alloc(nbytes)
            if off is None:
                self._release_lineages()
                off = self.heap.alloc(nbytes)
            if off is None:
                raise MemoryError(f"workspace exhausted: need {nbytes} bytes, largest free range {self.heap.largest_free}")
            blk = _Block(off, nbytes, stream, name)
        blk.stream, blk.name = stream, name
        t = self.buffer[blk.offset:blk.offset + n * torch.empty((), dtype=dtype).element_size()].view(dtype).view(*shape)
        self.live[t.data_ptr()] = blk
        if self._scopes:
            self._scopes[-1].append(t.data_ptr())
        self.peak = max(self.peak, self.heap.used)
        return t

    def free(self, t: torch.Tensor, stream: Optional[int] = None) -> None:
        blk = self.live.pop(t.data_ptr(), None)
        if blk is None:
            raise ValueError("tensor does not belong to this workspace (or was freed already)")
        if t.data_ptr() in self.frozen:
            self.live[t.data_ptr()] = blk
            return
        blk.stream = blk.stream if stream is None else stream
        self.free_by_stream.setdefault(blk.stream, []).append(blk)

    def promote(self, stream: int) -> None:
        """The caller guarantees that later work waits for `stream`: its free blocks return to the shared heap."""
        for b in self.free_by_stream.pop(stream, []):
            self.heap.free(b.offset)

    def _release_lineages(self) -> None:
        for s in list(self.free_by_stream):
            self.promote(s)

    # -- lifetime ----------------------------------------------------------------------------------------------
    def freeze(self) -> None:
        self.frozen.update(self.live.keys())

    @contextmanager
    def scope(self) -> Iterator["Workspace"]:
        self._scopes.append([])
        try:
            yield self
        finally:
            for ptr in self._scopes.pop():
                blk = self.live.get(ptr)
                if blk is not None and ptr not in self.frozen:
                    del self.live[ptr]
                    self.free_by_stream.setdefault(blk.stream, []).append(blk)

    def reset(self) -> None:
        for ptr in [p for p in self.live if p not in self.frozen]:
            self.heap.free(self.live.pop(ptr).offset)
        self._release_lineages()

    @property
    def used(self) -> int:
        return self.heap.used

    def layout(self) -> List[Tuple[str, int, int]]:
        """(name, offset, nbytes) of the live allocations: what a process that maps the arena over IPC needs."""
        return sorted(((b.name, b.offset, b.nbytes) for b in self.live.values()), key=lambda x: x[1])


class UsingHolder(Generic[T]):
    """A slot that owns one disposable value: `replace` disposes the previous one, leaving the `with` block
    disposes the last (reference `src/using-holder.ts`)."""

    def __init__(self, value: Optional[T] = None, dispose: Optional[Callable[[T], None]] = None):
        self.value = value
        self._dispose = dispose or (lambda v: getattr(v, "dispose", lambda: None)())

    def replace(self, value: Optional[T]) -> Optional[T]:
        if self.value is not None and self.value is not value:
            self._dispose(self.value)
        self.value = value
        return value

    def detach(self) -> Optional[T]:
        v, self.value = self.value, None
        return v

    def __enter__(self) -> "UsingHolder[T]":
        return self

    def __exit__(self, *exc) -> None:
        self.replace(None)


def walk_tensors(tree: Any, fn: Callable[[torch.Tensor], None]) -> None:
    """Apply `fn` to every tensor inside nested lists / tuples / dicts / dataclass-like objects
    (reference `src/tensor-tree.ts`: keep or dispose whole result structures)."""
    if isinstance(tree, torch.Tensor):
        fn(tree)
    elif isinstance(tree, dict):
        for v in tree.values():
            walk_tensors(v, fn)
    elif isinstance(tree, (list, tuple)):
        for v in tree:
            walk_tensors(v, fn)
    elif hasattr(tree, "__dict__") and not isinstance(tree, type):
        for v in vars(tree).values():
            walk_tensors(v, fn)
