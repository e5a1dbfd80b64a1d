"""Dense grouped-query attention over a paged bf16 KV cache and FP8 block-scaled linears
(Qwen3 / Qwen3.5 full-attention layers).

On CUDA the work runs in the sm_100a kernels of `csrc/dense_attn.cu`; on CPU the same
functions run the plain fp32 definition, which is also what the GPU tests compare against.
Reference counterparts: `fusedNormRope`, `kvCacheWrite`, `flashDecode`, `flashPrefillPaged`
(`src/execution-workspace.ts:392-814`, `csrc/glm_flash.cu`).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import reference as R


def _native():
    from . import native as N
    return N


class NormRopeParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("ldq", C.c_int), ("k", C.c_void_p), ("ldk", C.c_int), ("v", C.c_void_p), ("ldv", C.c_int),
                ("q_norm_w", C.c_void_p), ("k_norm_w", C.c_void_p), ("positions", C.c_void_p), ("batch_idx", C.c_void_p),
                ("page_table", C.c_void_p), ("pt_stride", C.c_int), ("page_size", C.c_int), ("n_heads", C.c_int),
                ("n_kv", C.c_int), ("hd", C.c_int), ("q_stride", C.c_int), ("rope_dim", C.c_int), ("eps", C.c_float),
                ("theta", C.c_float), ("q_out", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p)]


class AttnParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("positions", C.c_void_p),
                ("batch_idx", C.c_void_p), ("page_table", C.c_void_p), ("pt_stride", C.c_int), ("page_size", C.c_int),
                ("qo_indptr", C.c_void_p), ("n_heads", C.c_int), ("n_kv", C.c_int), ("hd", C.c_int), ("sm_scale", C.c_float),
                ("out", C.c_void_p), ("o_part", C.c_void_p), ("lse_part", C.c_void_p), ("splits", C.c_int)]


def _slots(positions, batch_idx, page_table, page_size):
    pages = page_table[batch_idx.long(), (positions // page_size).long()].long()
    return pages * page_size + (positions % page_size).long()


def qk_norm_rope_cache(q, k, v, q_norm_w, k_norm_w, positions, batch_idx, page_table, page_size, k_cache, v_cache,
                       n_heads: int, n_kv: int, hd: int, rope_dim: int, theta: float, eps: float, q_stride: Optional[int] = None):
    """Per-head RMSNorm (weights may be None) + rotate-half RoPE on q and k; k and v rows go into
    their cache slots.  q [T, n_heads * q_stride] (head h starts at h * q_stride), k/v
    [T, n_kv * hd]; caches [slots, n_kv, hd].  Returns q_out [T, n_heads, hd]."""
    T = q.shape[0]
    q_stride = hd if q_stride is None else q_stride
    if q.is_cuda:
        N = _native()
        q_out = torch.empty(T, n_heads, hd, dtype=torch.bfloat16, device=q.device)
        p = NormRopeParams(q=q.data_ptr(), ldq=q.stride(0), k=k.data_ptr(), ldk=k.stride(0), v=v.data_ptr(), ldv=v.stride(0),
                           q_norm_w=N.ptr(q_norm_w), k_norm_w=N.ptr(k_norm_w), positions=positions.data_ptr(),
                           batch_idx=batch_idx.data_ptr(), page_table=page_table.data_ptr(), pt_stride=page_table.stride(0),
                           page_size=page_size, n_heads=n_heads, n_kv=n_kv, hd=hd, q_stride=q_stride, rope_dim=rope_dim,
                           eps=eps, theta=theta, q_out=q_out.data_ptr(), k_cache=k_cache.data_ptr(), v_cache=v_cache.data_ptr())
        N.call("sl_qk_norm_rope_cache", C.byref(p), T, N.stream())
        return q_out
    qh = q.view(T, n_heads, q_stride)[..., :hd].to(torch.float32)
    kh = k.reshape(T, n_kv, hd).to(torch.float32)
    if q_norm_w is not None:
        qh = R.rmsnorm(qh, q_norm_w, eps).to(torch.bfloat16).to(torch.float32)
    if k_norm_w is not None:
        kh = R.rmsnorm(kh, k_norm_w, eps).to(torch.bfloat16).to(torch.float32)
    qh = R.apply_rope(qh, positions, theta, rope_dim, interleave=False)
    kh = R.apply_rope(kh, positions, theta, rope_dim, interleave=False)
    slots = _slots(positions, batch_idx, page_table, page_size)
    k_cache[slots] = kh.to(k_cache.dtype)
    v_cache[slots] = v.reshape(T, n_kv, hd).to(v_cache.dtype)
    return qh.to(q.dtype)


def _splits(T: int, n_kv: int, max_len: int) -> int:
    want = max(1, (148 * 2) // max(1, T * n_kv))
    return int(max(1, min(want, max(1, max_len // 128), 32)))


def paged_attention(q, k_cache, v_cache, positions, batch_idx, page_table, page_size, sm_scale: float,
                    qo_indptr: Optional[torch.Tensor] = None, max_q: int = 0, max_kv_len: int = 0):
    """Causal attention of each query token (absolute position positions[t], sequence row
    batch_idx[t]) over the cached keys 0..position of its sequence.  q [T, n_heads, hd] ->
    [T, n_heads, hd].  With `qo_indptr` ([B+1], contiguous query ranges per sequence) the
    tensor-core prefill kernel is used, otherwise split-KV decoding (one token per sequence)."""
    T, n_heads, hd = q.shape
    n_kv = k_cache.shape[1]
    if q.is_cuda:
        N = _native()
        p = AttnParams(q=q.data_ptr(), k_cache=k_cache.data_ptr(), v_cache=v_cache.data_ptr(), positions=positions.data_ptr(),
                       batch_idx=batch_idx.data_ptr(), page_table=page_table.data_ptr(), pt_stride=page_table.stride(0),
                       page_size=page_size, qo_indptr=N.ptr(qo_indptr), n_heads=n_heads, n_kv=n_kv, hd=hd, sm_scale=sm_scale)
        if qo_indptr is not None:
            out = torch.empty(T, n_heads, hd, dtype=torch.bfloat16, device=q.device)
            p.out = out.data_ptr()
            N.call("sl_paged_attn_prefill", C.byref(p), qo_indptr.numel() - 1, int(max_q or T), N.stream())
            return out
        splits = _splits(T, n_kv, max(1, max_kv_len))
        o_part = torch.empty(T, n_heads, splits, hd, dtype=torch.float32, device=q.device)
        lse_part = torch.empty(T, n_heads, splits, dtype=torch.float32, device=q.device)
        p.o_part, p.lse_part, p.splits = o_part.data_ptr(), lse_part.data_ptr(), splits
        N.call("sl_paged_attn_decode", C.byref(p), T, N.stream())
        out = torch.empty(T, n_heads, hd, dtype=torch.bfloat16, device=q.device)
        cp = N.CombineParams(n_buf=1, parts_per_buf=splits, h=n_heads, R=hd, head_begin=0, head_count=n_heads,
                             o_out=out.data_ptr(), lse_out=0, out_f32=0)
        cp.o_ptrs[0] = o_part.data_ptr()
        cp.lse_ptrs[0] = lse_part.data_ptr()
        N.call("sl_mla_combine", C.byref(cp), T, N.stream())
        return out
    out = torch.empty(T, n_heads, hd, dtype=torch.float32, device=q.device)
    for t in range(T):
        pos = int(positions[t])
        kp = torch.arange(pos + 1, device=q.device)
        slots = _slots(kp, torch.full_like(kp, int(batch_idx[t])), page_table, page_size)
        out[t] = R.dense_attention(q[t:t + 1], k_cache[slots], v_cache[slots], sm_scale, causal_offset=pos)[0]
    return out.to(q.dtype)


# ---- FP8 block-scaled weights (Qwen3-FP8: e4m3 weight + `weight_scale_inv` per 128x128 block) -----------------

def fp8_block_dequant(w8: torch.Tensor, scale_inv: torch.Tensor, block: int = 128) -> torch.Tensor:
    """w8 [N, K] float8_e4m3fn (or its uint8 bytes), scale_inv [ceil(N/b), ceil(K/b)] -> bf16 [N, K].
    Reference: `fp8_block_dequant_*` GEMV/GEMM family (`csrc/glm_gemv.cu`), expanded once at load
    here so that the bf16 tensor-core kernels serve these checkpoints."""
    from .quant import fp8_block_dequantize
    return fp8_block_dequantize(w8, scale_inv, block).to(torch.bfloat16)


def fp8_block_quantize(w: torch.Tensor, block: int = 128):
    """Inverse of :func:`fp8_block_dequant` (test fixtures, `csrc/glm_quantize.cu:1-73` for activations)."""
    N_, K = w.shape
    nb, kb = -(-N_ // block), -(-K // block)
    wp = torch.zeros(nb * block, kb * block, dtype=torch.float32, device=w.device)
    wp[:N_, :K] = w.to(torch.float32)
    blocks = wp.view(nb, block, kb, block)
    amax = blocks.abs().amax(dim=(1, 3)).clamp(min=1e-12)
    scale = amax / 448.0
    q = (blocks / scale.view(nb, 1, kb, 1)).clamp(-448, 448).view(nb * block, kb * block)[:N_, :K]
    return q.to(torch.float8_e4m3fn), scale
