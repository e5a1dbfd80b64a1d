"""Small stand-alone ops: FP8 activation quantisation, L2 prefetch, gather of selected KV rows.
CUDA tensors run the kernels of `csrc/quantize.cu` / `csrc/gather_ckv.cu`; CPU tensors run the
PyTorch definition (the oracle of the GPU tests)."""
from __future__ import annotations

import torch

from . import quant


def _native():
    from . import native as N
    return N


def quantize_fp8(x: torch.Tensor):
    """x [rows, K] -> (e4m3 bytes [rows, K] uint8, scales [rows, ceil(K/128)] fp32), one power-of-two scale
    per 128 values (reference `csrc/glm_quantize.cu`)."""
    rows, K = x.shape
    if x.is_cuda:
        N = _native()
        xb = x.to(torch.bfloat16).contiguous()
        q = torch.empty(rows, K, dtype=torch.uint8, device=x.device)
        s = torch.empty(rows, (K + 127) // 128, dtype=torch.float32, device=x.device)
        N.call("sl_quantize_fp8", q.data_ptr(), s.data_ptr(), xb.data_ptr(), rows, K, N.stream())
        return q, s
    pad = (-K) % 128
    xp = torch.nn.functional.pad(x.to(torch.bfloat16).to(torch.float32), (0, pad))
    q, s = quant.fp8_quantize_block(xp, 128, pow2=True)
    return q.view(torch.uint8)[:, :K].contiguous(), s


def prefetch_l2(t: torch.Tensor, stream=None) -> None:
    """Pull a tensor's bytes into L2 (no-op on CPU).  Launch it on a side stream ahead of the consumer."""
    if not t.is_cuda:
        return
    N = _native()
    s = N.stream() if stream is None else stream.cuda_stream
    N.call("sl_prefetch_l2", t.data_ptr(), t.numel() * t.element_size(), s)


class PrefetchSet:
    """Byte ranges of several tensors, packed once for `sl_prefetch_l2_multi` (at most 12 tensors; CPU tensors and
    None are skipped).  `launch(stream)` issues one kernel that pulls them all into L2."""

    def __init__(self, tensors, keep: bool = True):
        import ctypes as C
        ts = [t for t in tensors if t is not None and t.is_cuda and t.numel() > 0][:12]
        self.tensors = ts                                    # keeps the storage alive
        self.count = len(ts)
        self.keep = int(keep)
        self.nbytes = sum(t.numel() * t.element_size() for t in ts)
        self._ptrs = (C.c_void_p * max(1, self.count))(*[t.data_ptr() for t in ts])
        self._bytes = (C.c_ulonglong * max(1, self.count))(*[t.numel() * t.element_size() for t in ts])

    def launch(self, stream=None) -> None:
        if self.count == 0:
            return
        N = _native()
        s = N.stream() if stream is None else stream.cuda_stream
        N.call("sl_prefetch_l2_multi", self._ptrs, self._bytes, self.count, self.keep, s)


def gather_topk_ckv(kv_cache: torch.Tensor, slots: torch.Tensor, lengths: torch.Tensor, R: int, Dr: int, group: int):
    """Distinct selected rows of the packed cache as dense bf16 [U, R + Dr] (ascending slot order) and the
    fan-out table where[t, j] = row of slots[t, j] in that buffer (-1 for unused entries).
    Returns (dense, where, num_unique)."""
    T, k = slots.shape
    num_slots = kv_cache.shape[0]
    dev = kv_cache.device
    if kv_cache.is_cuda:
        N = _native()
        flags = torch.zeros(num_slots, dtype=torch.int32, device=dev)
        N.call("sl_gather_mark", flags.data_ptr(), slots.data_ptr(), lengths.data_ptr(), T, k, N.stream())
        incl = torch.cumsum(flags, 0, dtype=torch.int32)
        index = (incl - flags).contiguous()
        U = int(incl[-1]) if num_slots else 0
        dense = torch.empty(U, R + Dr, dtype=torch.bfloat16, device=dev)
        N.call("sl_gather_rows", dense.data_ptr(), kv_cache.data_ptr(), flags.data_ptr(), index.data_ptr(), num_slots, R, Dr, group,
               N.stream())
        where = torch.empty(T, k, dtype=torch.int32, device=dev)
        N.call("sl_gather_fanout", where.data_ptr(), slots.data_ptr(), lengths.data_ptr(), index.data_ptr(), T, k, N.stream())
        return dense, where, U
    valid = (torch.arange(k).unsqueeze(0) < lengths.unsqueeze(1)) & (slots >= 0)
    uniq = torch.unique(slots[valid].to(torch.int64))
    ckv, kpe = quant.unpack_kv_rows(kv_cache[uniq], R, Dr, group)
    dense = torch.cat([ckv, kpe], dim=1).to(torch.bfloat16)
    lookup = torch.full((num_slots,), -1, dtype=torch.int32)
    lookup[uniq] = torch.arange(uniq.numel(), dtype=torch.int32)
    where = torch.where(valid, lookup[slots.clamp(min=0).to(torch.int64)], torch.full_like(slots, -1)).to(torch.int32)
    return dense, where, int(uniq.numel())
