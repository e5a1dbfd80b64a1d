// Shared between the index scoring kernels (`indexer.cu`: FP8 `mma.sync` per-token / 8-token kernels;
// `indexer_tcgen05.cu`: prefill scorer on tcgen05 `kind::f8f6f4`).
#pragma once
#include "common.cuh"

struct IndexerScoreParams {
    const uint8_t* q8;        // [T, Hi, D] e4m3
    const float* w_eff;       // [T, Hi]
    const uint8_t* idx_cache; // [slots, D + 4]
    const int* page_table; int pt_stride;
    const int* batch_idx; const int* positions;
    int Hi, D, page_size, cp_world, cp_rank, top_k;
    float* scores; int ld_scores;     // [T, ld_scores]
    int num_slots;                    // rows of idx_cache (0 = unknown: no check)
    int* guard;                       // index self-check record (see guard_ok), may be null
    int one_sequence;                 // all T rows belong to one sequence (one page table): the prefill tensor-core scorer's case
    int* err;                         // error word of the bounded waits (tcgen05 scorer), may be null
};

// Visible local keys of a query at global position p: local key j is global j*W + r.
__device__ __forceinline__ int local_visible(int p, int W, int r) { return p >= r ? (p - r) / W + 1 : 0; }

// Prefill scorer on the 5th-generation tensor cores; returns -2 when the shape or alignment is not one it takes (the
// caller then uses the mma.sync kernels), 0 or a CUDA error otherwise.
int indexer_scores_tcgen05(const IndexerScoreParams* p, int T, int max_local, cudaStream_t s);
