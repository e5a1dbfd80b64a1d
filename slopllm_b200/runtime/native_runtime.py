"""Python faces of the host-side C++ runtime (`csrc/runtime/*.cpp`)."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

from ..ops import native as N

_U64_MAX = (1 << 64) - 1


def _lib():
    lib = N.runtime()
    if not getattr(lib, "_sl_typed", False):
        lib.rt_pool_create.restype = C.c_void_p
        lib.rt_pool_create.argtypes = [C.c_int]
        lib.rt_pool_destroy.argtypes = [C.c_void_p]
        for f in ("rt_pool_free_count",):
            getattr(lib, f).argtypes = [C.c_void_p]
        lib.rt_pool_alloc.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int32)]
        for f in ("rt_pool_ref", "rt_pool_unref", "rt_pool_refcount"):
            getattr(lib, f).argtypes = [C.c_void_p, C.c_int]
        lib.rt_common_prefix.restype = C.c_int64
        lib.rt_common_prefix.argtypes = [C.POINTER(C.c_int64), C.c_int64, C.POINTER(C.c_int64), C.c_int64]
        lib.rt_heap_create.restype = C.c_void_p
        lib.rt_heap_create.argtypes = [C.c_uint64, C.c_uint64]
        lib.rt_heap_destroy.argtypes = [C.c_void_p]
        lib.rt_heap_alloc.restype = C.c_uint64
        lib.rt_heap_alloc.argtypes = [C.c_void_p, C.c_uint64]
        lib.rt_heap_free.argtypes = [C.c_void_p, C.c_uint64]
        lib.rt_heap_used.restype = C.c_uint64
        lib.rt_heap_used.argtypes = [C.c_void_p]
        lib.rt_heap_largest_free.restype = C.c_uint64
        lib.rt_heap_largest_free.argtypes = [C.c_void_p]
        lib.rt_heap_num_free_ranges.argtypes = [C.c_void_p]
        lib.rt_mmap_open.restype = C.c_void_p
        lib.rt_mmap_open.argtypes = [C.c_char_p, C.POINTER(C.c_uint64)]
        lib.rt_mmap_close.argtypes = [C.c_void_p]
        lib.rt_mmap_advise.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64]
        lib.rt_mmap_copy_rows.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p, C.c_int]
        lib._sl_typed = True
    return lib


class PagePool:
    """Free list + refcounts of KV pages."""

    def __init__(self, num_pages: int):
        self._lib = _lib()
        self._h = self._lib.rt_pool_create(num_pages)
        self.num_pages = num_pages

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.rt_pool_destroy(self._h)
            self._h = None

    def free_count(self) -> int:
        return self._lib.rt_pool_free_count(self._h)

    def alloc(self, n: int) -> Optional[List[int]]:
        buf = (C.c_int32 * n)()
        if self._lib.rt_pool_alloc(self._h, n, buf) != 0:
            return None
        return list(buf)

    def ref(self, page: int) -> int:
        return self._lib.rt_pool_ref(self._h, page)

    def unref(self, page: int) -> int:
        return self._lib.rt_pool_unref(self._h, page)

    def refcount(self, page: int) -> int:
        return self._lib.rt_pool_refcount(self._h, page)


class Heap:
    """First-fit range allocator with coalescing (offsets into an arena)."""

    def __init__(self, capacity: int, alignment: int = 256):
        self._lib = _lib()
        self._h = self._lib.rt_heap_create(capacity, alignment)
        self.capacity = capacity

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.rt_heap_destroy(self._h)
            self._h = None

    def alloc(self, size: int) -> Optional[int]:
        off = self._lib.rt_heap_alloc(self._h, size)
        return None if off == _U64_MAX else off

    def free(self, offset: int) -> None:
        if self._lib.rt_heap_free(self._h, offset) != 0:
            raise ValueError(f"offset {offset} is not a live allocation")

    @property
    def used(self) -> int:
        return self._lib.rt_heap_used(self._h)

    @property
    def largest_free(self) -> int:
        return self._lib.rt_heap_largest_free(self._h)

    @property
    def num_free_ranges(self) -> int:
        return self._lib.rt_heap_num_free_ranges(self._h)


class MappedFile:
    """Read-only mapping of a checkpoint shard in the C++ runtime (`csrc/runtime/mmap_loader.cpp`): strided windows are
    copied into a caller-provided buffer (normally pinned host memory) by several threads."""

    def __init__(self, path: str):
        size = C.c_uint64(0)
        self._h = _lib().rt_mmap_open(path.encode(), C.byref(size))
        if not self._h:
            raise OSError(f"cannot map {path}")
        self.path, self.size = path, int(size.value)

    def advise(self, offset: int, length: int) -> None:
        """Start reading a range ahead of its use (MADV_WILLNEED)."""
        _lib().rt_mmap_advise(self._h, offset, length)

    def copy_rows(self, offset: int, row_stride: int, row_bytes: int, rows: int, dst_ptr: int, threads: int = 4) -> None:
        """dst[r * row_bytes ...] = file[offset + r * row_stride ...] for r < rows."""
        rc = _lib().rt_mmap_copy_rows(self._h, offset, row_stride, row_bytes, rows, dst_ptr, threads)
        if rc != 0:
            raise ValueError(f"{self.path}: window (offset {offset}, {rows} rows of {row_bytes} bytes every {row_stride}) "
                             f"is outside the file of {self.size} bytes")

    def close(self) -> None:
        if self._h:
            _lib().rt_mmap_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001  (interpreter shutdown)
            pass
