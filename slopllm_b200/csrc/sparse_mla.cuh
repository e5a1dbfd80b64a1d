// Arguments of the sparse MLA split kernels (tensor-core forms); the ctypes mirror is `SparseMlaParams`
// (`ops/native.py`).  The scalar kernel (csrc/sparse_mla.cu) reads a prefix of the same layout.
#pragma once

#include "common.cuh"

struct SparseMlaParams {
    const bf16* q_abs;        // [T, h, R]
    const bf16* q_pe;         // [T, h, Dr]
    const uint8_t* kv_cache;  // [slots, row_bytes]
    const int* slots;         // [T, topk]
    const int* lengths;       // [T]
    int h, R, Dr, group, topk, splits;
    float sm_scale;
    float* o_part;            // [T, h, splits, R]
    float* lse_part;          // [T, h, splits]
    int num_slots;            // rows of kv_cache (0 = unknown: no check)
    int* guard;               // index self-check record (see guard_ok), may be null
    bf16* o_final;            // keys-on-M kernels with splits == 1: final output [T, h, R] (then o_part / lse_part are not written)
    float* lse_final;         // [T, h], may be null
    int* err;                 // error word of the tcgen05 kernels (bounded waits), may be null: then the mma.sync kernels run
};

// Prefill form on tcgen05 (csrc/sparse_mla_tcgen05.cu).  Returns -2 when the launch is not one it covers
// (the caller then takes the mma.sync kernels), else the launch status.
int sparse_mla_tcgen05(const SparseMlaParams* p, int T, cudaStream_t s);
