"""Number formats: NVFP4 (E2M1 + UE4M3 block scales + f32 global), FP8 E4M3 block quant.

These are the pure-torch definitions that every CUDA kernel is tested against.

NVFP4 layout (reference `csrc/glm_nvfp4.cuh:1-125`, `tests/python/test_nvfp4.py`):
``w = e2m1(nibble) * e4m3(scale[row, k // 16]) * scale_2``; two codes per byte, the
element with the even k index in the low nibble.
"""
from __future__ import annotations

import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
NVFP4_BLOCK = 16
FP8_MAX = 448.0
FP4_MAX = 6.0


def e2m1_table(device=None, dtype=torch.float32) -> torch.Tensor:
    """16-entry code -> value table (bit 3 is the sign)."""
    pos = torch.tensor(E2M1_VALUES, dtype=dtype, device=device)
    return torch.cat([pos, -pos])


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    """uint8 [..., K/2] -> int64 codes [..., K] (low nibble first)."""
    p = packed.to(torch.int64)
    lo, hi = p & 0xF, (p >> 4) & 0xF
    return torch.stack([lo, hi], dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """integer codes [..., K] -> uint8 [..., K/2]."""
    c = codes.to(torch.int64).reshape(*codes.shape[:-1], codes.shape[-1] // 2, 2)
    return (c[..., 0] | (c[..., 1] << 4)).to(torch.uint8)


def nvfp4_dequantize(packed: torch.Tensor, block_scale: torch.Tensor, global_scale,
                     dtype=torch.float32) -> torch.Tensor:
    """Dequantise NVFP4 `[..., N, K/2]` u8 + `[..., N, K/16]` e4m3 + f32 global scale."""
    vals = e2m1_table(packed.device)[unpack_nibbles(packed)]
    s = block_scale.to(torch.float32).repeat_interleave(NVFP4_BLOCK, dim=-1)
    g = torch.as_tensor(global_scale, dtype=torch.float32, device=packed.device)
    while g.dim() < vals.dim() and g.dim() > 0:
        g = g.unsqueeze(-1)
    return (vals * s * g).to(dtype)


def _round_to_e2m1_codes(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest (ties to even code) of |x| <= 6 onto the E2M1 grid -> 4-bit codes."""
    a = x.abs().clamp(max=FP4_MAX)
    # thresholds halfway between representable magnitudes; ties go to the even mantissa
    bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=x.device, dtype=x.dtype)
    idx = torch.bucketize(a, bounds, right=False)
    # exact ties: 0.25->0 (0.0), 0.75->2 (1.0), 1.25->2, 1.75->4 (2.0), 2.5->4, 3.5->6 (4.0), 5.0->6
    tie_up = torch.tensor([False, True, False, True, False, True, False], device=x.device)
    on_tie = (a.unsqueeze(-1) == bounds).any(-1)
    tie_idx = torch.bucketize(a, bounds, right=True) - 1
    bump = on_tie & tie_up[tie_idx.clamp(min=0)]
    idx = idx + bump.to(idx.dtype)
    return idx | ((x < 0).to(idx.dtype) << 3)


def nvfp4_quantize(w: torch.Tensor, global_scale=None):
    """Quantise `[..., N, K]` to NVFP4.  Returns (packed u8, e4m3 block scale, f32 global).

    The global scale defaults to ``amax / (448 * 6)`` so block scales use the e4m3 range.
    """
    w = w.to(torch.float32)
    K = w.shape[-1]
    assert K % NVFP4_BLOCK == 0
    if global_scale is None:
        amax = w.abs().amax().clamp(min=1e-12)
        global_scale = amax / (FP8_MAX * FP4_MAX)
    g = torch.as_tensor(global_scale, dtype=torch.float32, device=w.device)
    blocks = w.reshape(*w.shape[:-1], K // NVFP4_BLOCK, NVFP4_BLOCK)
    bmax = blocks.abs().amax(-1)
    scale = (bmax / FP4_MAX / g).clamp(max=FP8_MAX).to(torch.float8_e4m3fn)
    sf = scale.to(torch.float32) * g
    q = blocks / sf.clamp(min=1e-30).unsqueeze(-1)
    codes = _round_to_e2m1_codes(q).reshape(*w.shape)
    return pack_nibbles(codes), scale, g.reshape(())


def nvfp4_fake_quant_rows(x: torch.Tensor) -> torch.Tensor:
    """What a row of activations becomes on the W4A4 path: NVFP4 with one global scale per row (amax / (6 * 448)), e4m3
    scales per 16 values, E2M1 codes, back in fp32 (the definition `sl_nvfp4_quantize_rows` is tested against)."""
    xf = x.to(torch.float32)
    K = xf.shape[-1]
    g = (xf.abs().amax(-1, keepdim=True) / (FP8_MAX * FP4_MAX))
    g = torch.where(g > 0, g, torch.ones_like(g))
    blocks = xf.reshape(*xf.shape[:-1], K // NVFP4_BLOCK, NVFP4_BLOCK)
    scale = (blocks.abs().amax(-1) / FP4_MAX / g).to(torch.float8_e4m3fn).to(torch.float32)
    dq = (scale * g).unsqueeze(-1)
    codes = _round_to_e2m1_codes(torch.where(dq > 0, blocks / dq.clamp(min=1e-30), torch.zeros_like(blocks)))
    return (e2m1_table(x.device)[codes] * dq).reshape(xf.shape)


def fp8_quantize_block(x: torch.Tensor, block: int = 128, pow2: bool = False):
    """Per-`block` e4m3 quantisation along the last dim.  Returns (fp8 tensor, f32 scales).

    ``pow2=False`` is the packed-KV rule (scale = max(amax/448, FLT_MIN), reference
    `csrc/glm_flash.cu:1081-1133`); ``pow2=True`` rounds the scale up to a power of two
    with ``amax`` floored at 1e-4 (indexer K rows, `csrc/glm_indexer_cache.cuh:9-16`;
    also `csrc/glm_quantize.cu:8`).
    """
    xf = x.to(torch.float32)
    K = xf.shape[-1]
    assert K % block == 0
    b = xf.reshape(*xf.shape[:-1], K // block, block)
    amax = b.abs().amax(-1)
    if pow2:
        raw = amax.clamp(min=1e-4) / FP8_MAX
        scale = torch.exp2(torch.ceil(torch.log2(raw)))
    else:
        scale = (amax / FP8_MAX).clamp(min=torch.finfo(torch.float32).tiny)
    q = (b / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(x.shape), scale


def fp8_dequantize_block(q: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    qf = q.to(torch.float32)
    K = qf.shape[-1]
    return (qf.reshape(*qf.shape[:-1], K // block, block) * scale.unsqueeze(-1)).reshape(qf.shape)


# ---- packed sparse-MLA cache rows -------------------------------------------------------

def fp8_block_dequantize(w8: torch.Tensor, scale_inv: torch.Tensor, block: int = 128) -> torch.Tensor:
    """FP8 weight matrix w8 [N, K] (float8_e4m3fn or its bytes) with one scale per block x block tile
    (scale_inv [ceil(N/block), ceil(K/block)]) -> fp32 [N, K]."""
    if w8.dtype == torch.uint8:
        w8 = w8.view(torch.float8_e4m3fn)
    n, k = w8.shape
    s = scale_inv.to(torch.float32).repeat_interleave(block, 0)[:n].repeat_interleave(block, 1)[:, :k]
    return w8.to(torch.float32) * s


def pack_kv_rows(ckv: torch.Tensor, kpe: torch.Tensor, group: int = 128) -> torch.Tensor:
    """[T, R] latent + [T, Dr] rope key -> u8 rows `[T, R + 4*R/group + 2*Dr]`.

    Row = R e4m3 bytes | R/group f32 scales | Dr bf16 rope values
    (reference `csrc/glm_flash.cu:1136-1230`; 656 B for R=512, Dr=64).
    """
    q, scale = fp8_quantize_block(ckv.to(torch.bfloat16), group)
    parts = [q.view(torch.uint8), scale.contiguous().view(torch.uint8).reshape(ckv.shape[0], -1),
             kpe.to(torch.bfloat16).contiguous().view(torch.uint8).reshape(kpe.shape[0], -1)]
    return torch.cat(parts, dim=-1)


def unpack_kv_rows(rows: torch.Tensor, kv_lora: int, rope_dim: int, group: int = 128):
    """Inverse of :func:`pack_kv_rows` -> (ckv f32 [T, R], kpe f32 [T, Dr])."""
    ng = kv_lora // group
    q = rows[..., :kv_lora].contiguous().view(torch.float8_e4m3fn)
    scale = rows[..., kv_lora:kv_lora + 4 * ng].contiguous().view(torch.float32)
    kpe = rows[..., kv_lora + 4 * ng:].contiguous().view(torch.bfloat16)
    return fp8_dequantize_block(q, scale, group), kpe.to(torch.float32)


def pack_index_rows(k: torch.Tensor) -> torch.Tensor:
    """Indexer key rows `[T, D]` -> u8 `[T, D + 4]`: D e4m3 bytes | one power-of-two f32 scale."""
    q, scale = fp8_quantize_block(k.to(torch.bfloat16), k.shape[-1], pow2=True)
    return torch.cat([q.view(torch.uint8), scale.contiguous().view(torch.uint8).reshape(k.shape[0], 4)], -1)


def unpack_index_rows(rows: torch.Tensor, dim: int) -> torch.Tensor:
    q = rows[..., :dim].contiguous().view(torch.float8_e4m3fn).to(torch.float32)
    scale = rows[..., dim:dim + 4].contiguous().view(torch.float32)
    return q * scale


# ---- random NVFP4 weights (benchmark / test initialisation) -------------------------------

def random_nvfp4(shape, generator: torch.Generator, device="cpu", scale_mult: float = 1.0 / 64):
    """Random-init NVFP4 tensor of logical shape `[..., N, K]`.

    E2M1 codes uniform over the 16 codes; E4M3 block scales log-normal(0, 0.5) * `scale_mult`;
    f32 global scale 1.0.
    """
    *lead, n, k = shape
    codes = torch.randint(0, 256, (*lead, n, k // 2), generator=generator, device=device, dtype=torch.uint8)
    s = torch.empty((*lead, n, k // NVFP4_BLOCK), device=device, dtype=torch.float32)
    s.normal_(0.0, 0.5, generator=generator).exp_().mul_(scale_mult)
    return codes, s.to(torch.float8_e4m3fn), torch.ones((), dtype=torch.float32, device=device)
