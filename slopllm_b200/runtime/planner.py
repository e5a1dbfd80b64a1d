"""Launch planning that depends only on shapes (reference: `src/sparse-mla-planner.ts:1-21`,
`sparseMlaChunksPerBlock`)."""
from __future__ import annotations

import os

NUM_SMS = 148
# waves of sparse-MLA CTAs the key split aims for (2: about 300 CTAs for the 148 SMs x 2 resident CTAs)
MLA_WAVES = int(os.environ.get("SLOPLLM_B200_MLA_WAVES", "2"))


def sparse_mla_splits(tokens: int, heads: int, topk: int, heads_per_cta: int = 16, chunk: int = 64, waves: int = 0,
                      max_splits: int = 64) -> int:
    """Number of key splits for the sparse-MLA kernel: enough CTAs (tokens x head groups x splits) for `waves`
    waves over the SMs, never less than one 64-key chunk per split."""
    waves = waves or MLA_WAVES
    groups = (heads + heads_per_cta - 1) // heads_per_cta
    want = max(1, (NUM_SMS * waves) // max(1, tokens * groups))
    return int(max(1, min(want, max(1, topk // chunk), max_splits)))


def smallt_splits(tokens: int, features: int, reduction: int, bm: int = 128, bk: int = 64) -> int:
    """K splits of the swap-AB small-T linear (mirror of `sl_smallT_splits` in csrc/gemm_tcgen05.cu): two CTAs
    fit per SM, so the target is ~200 CTAs, at least four 64-wide K blocks per split."""
    ctas, total_kb = (features + bm - 1) // bm, (reduction + bk - 1) // bk
    if tokens <= 0 or ctas >= 120 or total_kb < 8:
        return 1
    splits = min(8, (200 + ctas - 1) // ctas, total_kb // 4)
    per = (total_kb + splits - 1) // splits
    return max(1, (total_kb + per - 1) // per)


def padded_kv_len(n: int) -> int:
    """Decode graphs are keyed by this bucket of the longest sequence: max(1024, next power of two)
    (reference `src/execution-workspace.ts:553-646`)."""
    p = 1024
    while p < n:
        p <<= 1
    return p
