"""ctypes binding of the in-tree native libraries.

`kernels()` returns the CUDA kernel library (`_lib/libslopllm_kernels.so`, built by
`slopllm_b200.build_native` for sm_100a) and raises if it is missing: on a GPU box there is
no silent PyTorch fallback.  The reference binds its `libglm_ops.so` the same way in its
kernel tests (`tests/python/helpers.py`).
"""
from __future__ import annotations

import ctypes as C
import os
from functools import lru_cache

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(os.path.dirname(_HERE), "_lib")
KERNELS_SO = os.path.join(LIB_DIR, "libslopllm_kernels.so")
RUNTIME_SO = os.path.join(LIB_DIR, "libslopllm_runtime.so")

vp, i32, f32, u32, i64 = C.c_void_p, C.c_int, C.c_float, C.c_uint32, C.c_longlong


class NativeError(RuntimeError):
    pass


class CollectiveTimeout(RuntimeError):
    """A device-side bounded wait expired (a peer did not publish its flag in time)."""


@lru_cache(maxsize=None)
def kernels() -> C.CDLL:
    if not os.path.exists(KERNELS_SO):
        raise NativeError(f"{KERNELS_SO} is missing: run `python -m slopllm_b200.build_native` "
                          "(the CUDA path has no PyTorch fallback)")
    lib = C.CDLL(os.environ.get("SLOPLLM_B200_KERNELS_SO", KERNELS_SO))
    # programmatic dependent launch between the library's kernels; SLOPLLM_B200_PDL=0 turns it off
    lib.sl_set_pdl.argtypes = [i32]
    lib.sl_set_pdl.restype = None
    lib.sl_set_pdl(0 if os.environ.get("SLOPLLM_B200_PDL", "1") == "0" else 1)
    lib.sl_indexer_set_tiled.argtypes = [i32]
    lib.sl_indexer_set_tiled.restype = None
    lib.sl_indexer_set_tiled(0 if os.environ.get("SLOPLLM_B200_INDEXER_TILED", "1") == "0" else 1)
    lib.sl_indexer_set_tcgen05.argtypes = [i32]
    lib.sl_indexer_set_tcgen05.restype = None
    lib.sl_indexer_set_tcgen05(0 if os.environ.get("SLOPLLM_B200_INDEXER_TCGEN05", "1") == "0" else 1)
    lib.sl_sparse_mla_direct_ok.argtypes = [i32, i32, i32]
    lib.sl_sparse_mla_direct_ok.restype = i32
    lib.sl_sparse_mla_set_transposed.argtypes = [i32]
    lib.sl_sparse_mla_set_transposed.restype = None
    lib.sl_sparse_mla_set_transposed(0 if os.environ.get("SLOPLLM_B200_MLA_TRANSPOSED", "1") == "0" else 1)
    lib.sl_sparse_mla_set_tcgen05.argtypes = [i32]
    lib.sl_sparse_mla_set_tcgen05.restype = None
    # SLOPLLM_B200_MLA_TCGEN05: 0 = mma.sync everywhere, prefill = tcgen05 only where the kernel writes the final output,
    # anything else (default) = also the key-split launches of decode
    lib.sl_sparse_mla_set_tcgen05({"0": 0, "prefill": 1}.get(os.environ.get("SLOPLLM_B200_MLA_TCGEN05", "1"), 3))
    lib.sl_sparse_mla_tcgen05_decode_ok.argtypes = [i32, i32, i32, i32, i32]
    lib.sl_sparse_mla_tcgen05_decode_ok.restype = i32
    return lib


@lru_cache(maxsize=None)
def runtime() -> C.CDLL:
    if not os.path.exists(RUNTIME_SO):
        from .. import build_native
        build_native.build_runtime()
    return C.CDLL(RUNTIME_SO)


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = f"{what} failed with code {rc}"
        if rc > 0:
            msg += f" (cudaError {rc})"
        raise NativeError(msg)


# ---- parameter structs (field order mirrors csrc/*.cu) --------------------------------------------


class AttnPreParams(C.Structure):
    _fields_ = [("qkv", vp), ("ld", i32), ("q_lora", i32), ("kv_lora", i32), ("rope_dim", i32), ("idx_dim", i32),
                ("idx_heads", i32), ("q_norm_w", vp), ("kv_norm_w", vp), ("idx_ln_w", vp), ("idx_ln_b", vp),
                ("eps", f32), ("theta", f32), ("rope_interleave", i32), ("idx_rope_interleave", i32),
                ("positions", vp), ("batch_idx", vp), ("page_table", vp), ("pt_stride", i32), ("page_size", i32),
                ("cp_world", i32), ("cp_rank", i32), ("kv_group", i32), ("kv_cache", vp), ("idx_cache", vp),
                ("cq_out", vp), ("idx_w_out", vp), ("n_slabs", i32), ("slab_stride", i64), ("num_slots", i32), ("guard", vp)]


class QPostParams(C.Structure):
    _fields_ = [("qb", vp), ("ld", i32), ("heads", i32), ("d_nope", i32), ("rope_dim", i32), ("idx_heads", i32),
                ("idx_dim", i32), ("theta", f32), ("rope_interleave", i32), ("idx_rope_interleave", i32),
                ("positions", vp), ("idx_w", vp), ("q_pe_out", vp), ("q8_out", vp), ("w_eff_out", vp), ("n_slabs", i32),
                ("slab_stride", i64)]


class IndexerScoreParams(C.Structure):
    _fields_ = [("q8", vp), ("w_eff", vp), ("idx_cache", vp), ("page_table", vp), ("pt_stride", i32),
                ("batch_idx", vp), ("positions", vp), ("Hi", i32), ("D", i32), ("page_size", i32), ("cp_world", i32),
                ("cp_rank", i32), ("top_k", i32), ("scores", vp), ("ld_scores", i32), ("num_slots", i32), ("guard", vp),
                ("one_sequence", i32), ("err", vp)]


class TopkSelectParams(C.Structure):
    _fields_ = [("scores", vp), ("ld_scores", i32), ("positions", vp), ("top_k", i32), ("cp_world", i32),
                ("cp_rank", i32), ("out_pos", vp), ("out_score", vp), ("slots", vp), ("lengths", vp),
                ("page_table", vp), ("batch_idx", vp), ("pt_stride", i32), ("page_size", i32), ("n_fixed", i32)]


class SparseMlaParams(C.Structure):
    _fields_ = [("q_abs", vp), ("q_pe", vp), ("kv_cache", vp), ("slots", vp), ("lengths", vp), ("h", i32), ("R", i32),
                ("Dr", i32), ("group", i32), ("topk", i32), ("splits", i32), ("sm_scale", f32), ("o_part", vp),
                ("lse_part", vp), ("num_slots", i32), ("guard", vp), ("o_final", vp), ("lse_final", vp), ("err", vp)]


class CombineParams(C.Structure):
    _fields_ = [("o_ptrs", vp * 8), ("lse_ptrs", vp * 8), ("n_buf", i32), ("parts_per_buf", i32), ("h", i32), ("R", i32),
                ("head_begin", i32), ("head_count", i32), ("o_out", vp), ("lse_out", vp), ("out_f32", i32), ("parity_epoch", vp),
                ("parity_o_stride", i64), ("parity_lse_stride", i64)]


class CombineExpandParams(C.Structure):
    _fields_ = [("o_part", vp), ("lse_part", vp), ("w_v", vp), ("y", vp), ("xp", vp), ("T", i32), ("tpad", i32), ("Hh", i32),
                ("K", i32), ("N", i32), ("np", i32)]


class MoeGateUpParams(C.Structure):
    _fields_ = [("x", vp), ("ldx", i32), ("ids", vp), ("T", i32), ("top_k", i32), ("H", i32), ("I", i32),
                ("expert_offset", i32), ("num_local", i32), ("w13", vp), ("s13", vp), ("g13", vp), ("sw13", vp),
                ("ss13", vp), ("sg13", vp), ("act", vp)]


class MoeDownParams(C.Structure):
    _fields_ = [("act", vp), ("ids", vp), ("wts", vp), ("T", i32), ("top_k", i32), ("H", i32), ("I", i32),
                ("expert_offset", i32), ("num_local", i32), ("w2", vp), ("s2", vp), ("g2", vp), ("sw2", vp), ("ss2", vp),
                ("sg2", vp), ("out", vp), ("out_f32", i32), ("accumulate", i32)]


class MoeGroupedArgs(C.Structure):
    _fields_ = [("x", vp), ("ldx", i32), ("ids", vp), ("wts", vp), ("T", i32), ("top_k", i32), ("H", i32), ("I", i32),
                ("expert_offset", i32), ("num_local", i32), ("w13", vp), ("s13", vp), ("g13", vp), ("sw13", vp), ("ss13", vp),
                ("sg13", vp), ("w2", vp), ("s2", vp), ("g2", vp), ("sw2", vp), ("ss2", vp), ("sg2", vp), ("xp", vp),
                ("act_perm", vp), ("y_route", vp), ("plan", vp), ("max_items", i32), ("out", vp), ("xp_ready", i32)]


class MoePersistArgs(C.Structure):
    _fields_ = [("x", vp), ("ldx", i32), ("xp", vp), ("router_w", vp), ("bias", vp), ("E", i32), ("n_group", i32),
                ("topk_group", i32), ("norm", i32), ("scale", f32), ("T", i32), ("top_k", i32), ("H", i32), ("I", i32),
                ("expert_offset", i32), ("num_local", i32), ("w13", vp), ("s13", vp), ("g13", vp), ("sw13", vp), ("ss13", vp),
                ("sg13", vp), ("w2", vp), ("s2", vp), ("g2", vp), ("sw2", vp), ("ss2", vp), ("sg2", vp), ("slabs", vp),
                ("act_perm", vp), ("y_route", vp), ("plan", vp), ("ids", vp), ("wts", vp), ("sync", vp), ("status", vp),
                ("out", vp), ("max_items", i32), ("gsub", i32), ("trace", vp)]


class MoeRouterArgs(C.Structure):
    _fields_ = [("router_w", vp), ("bias", vp), ("E", i32), ("n_group", i32), ("topk_group", i32), ("norm", i32),
                ("scale", f32), ("slabs", vp), ("counter", vp)]


class SampleParams(C.Structure):
    _fields_ = [("logits", vp), ("V", i32), ("ld", i32), ("temperature", vp), ("top_p", vp), ("rep_penalty", vp),
                ("presence_penalty", vp), ("top_k", vp), ("history", vp), ("hist_len", vp), ("window", i32),
                ("max_k", i32), ("counter", vp), ("stream", u32), ("row_ids", vp), ("out_token", vp), ("cand_ids", vp),
                ("cand_probs", vp)]


class SpecRejectParams(C.Structure):
    _fields_ = [("draft_tokens", vp), ("draft_ids", vp), ("draft_probs", vp), ("target_ids", vp), ("target_probs", vp),
                ("D", i32), ("C", i32), ("counter", vp), ("out_tokens", vp), ("num_accepted", vp)]


# ---- function signatures ----------------------------------------------------------------------------------

_SIGS = {
    "sl_embed": [vp, vp, vp, i32, i32, i32, vp],
    "sl_add_rmsnorm": [vp, vp, vp, vp, vp, i32, i32, f32, i32, vp, vp],
    "sl_attn_pre": [C.POINTER(AttnPreParams), i32, vp],
    "sl_q_post": [C.POINTER(QPostParams), i32, vp],
    "sl_q_post_absorb": [C.POINTER(QPostParams), vp, vp, i32, i32, vp],
    "sl_gemm_bf16_tcgen05_batched": [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp],
    "sl_bmv": [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i64, vp],
    "sl_smallT_splits": [i32, i32, i32],
    "sl_gather_fetch": [vp, vp, vp, i32, C.c_size_t, C.c_size_t, vp],
    "sl_quantize_fp8": [vp, vp, vp, i32, i32, vp],
    "sl_prefetch_l2": [vp, C.c_size_t, vp],
    "sl_prefetch_l2_multi": [vp, vp, i32, i32, vp],
    "sl_gather_mark": [vp, vp, vp, i32, i32, vp],
    "sl_gather_rows": [vp, vp, vp, vp, i32, i32, i32, i32, vp],
    "sl_gather_fanout": [vp, vp, vp, vp, i32, i32, vp],
    "sl_qk_norm_rope_cache": [vp, i32, vp],
    "sl_paged_attn_prefill": [vp, i32, i32, vp],
    "sl_paged_attn_decode": [vp, i32, vp],
    "sl_delta_scan": [vp, i32, vp],
    "sl_causal_conv1d": [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp],
    "sl_rmsnorm_gated": [vp, vp, vp, vp, i32, i32, f32, i32, vp],
    "sl_mhc_pre": [vp, vp, vp, vp, vp, vp, vp, i32, i32, f32, f32, i32, vp],
    "sl_mhc_post": [vp, vp, vp, vp, vp, i32, i32, vp],
    "sl_mhc_streams": [vp, vp, i32, i32, i32, vp],
    "sl_silu_mul": [vp, vp, i32, i32, vp],
    "sl_silu_mul_h": [vp, vp, i32, i32, vp],
    "sl_moe_sort_routes": [vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp],
    "sl_gather_rows_f16": [vp, vp, vp, i32, i32, i32, i32, vp],
    "sl_gemm_w4_tcgen05": [vp, vp, vp, vp, i32, i32, vp, i32, i32, i32, i32, i32, i32, vp, i32, vp],
    "sl_grouped_gemm_w4_tcgen05": [vp, vp, vp, vp, i32, i32, vp, i32, i32, i32, i32, i32, i32, vp, vp, i32, vp, i32, vp],
    "sl_route_topk": [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp],
    "sl_topk_to_slots": [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp, vp],
    "sl_rotate_input_ids": [vp, vp, vp, vp, i32, vp],
    "sl_gemv_bf16": [vp, vp, vp, i32, i32, i32, i32, i32, vp],
    "sl_gemv_nvfp4": [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp],
    "sl_moe_gate_up": [C.POINTER(MoeGateUpParams), vp],
    "sl_moe_down": [C.POINTER(MoeDownParams), vp],
    "sl_indexer_scores": [C.POINTER(IndexerScoreParams), i32, i32, vp],
    "sl_topk_select": [C.POINTER(TopkSelectParams), i32, vp],
    "sl_sparse_mla_split": [C.POINTER(SparseMlaParams), i32, vp],
    "sl_sparse_mla_split_mma": [C.POINTER(SparseMlaParams), i32, vp],
    "sl_mla_combine": [C.POINTER(CombineParams), i32, vp],
    "sl_combine_vexpand": [C.POINTER(CombineExpandParams), vp],
    "sl_argmax": [vp, vp, i32, i32, i32, i32, i64, vp, vp, vp, vp],
    "sl_sample": [C.POINTER(SampleParams), i32, vp],
    "sl_spec_reject": [C.POINTER(SpecRejectParams), i32, vp],
    "sl_advance_counter": [vp, u32, vp],
    "sl_moe_grouped_mma": [C.POINTER(MoeGroupedArgs), vp, vp, vp],
    "sl_moe_persist": [C.POINTER(MoePersistArgs), vp, vp],
    "sl_moe_persist_ok": [i32, i32, i32, i32, i32, i32, i32],
    "sl_permute_x": [vp, vp, i32, i32, i32, vp],
    "sl_moe_route_reduce": [vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp, vp],
    "sl_linear_nvfp4_mma": [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp],
    "sl_linear_smallT_bf16_tcgen05": [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp, vp, i32, vp],
    "sl_grouped_gemm_bf16_tcgen05": [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, i32, vp, i32, vp],
    "sl_build_group_tiles": [vp, vp, vp, i32, i32, i32, i32, vp],
    "sl_nvfp4_dequant_bf16": [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp],
    "sl_linear_fp8_block": [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp],
    "sl_fp8_block_dequant_bf16": [vp, vp, vp, i32, i32, i32, vp],
    "sl_moe_unsort_reduce": [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp],
    "sl_gemm_bf16_tcgen05": [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp, i32, vp],
}


@lru_cache(maxsize=None)
def fn(name: str):
    f = getattr(kernels(), name)
    f.argtypes = _SIGS[name]
    f.restype = i32
    return f


_launches = 0


def launch_count() -> int:
    """Number of native kernel-launching calls made so far by this process."""
    return _launches


def kernel_count() -> int:
    """Number of CUDA kernels the library has launched so far (one native call may launch several)."""
    f = kernels().sl_kernel_launches
    f.restype = C.c_ulonglong
    f.argtypes = []
    return int(f())


def call(name: str, *args) -> None:
    global _launches
    _launches += 1
    check(fn(name)(*args), name)
