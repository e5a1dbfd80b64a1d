// Gather the selected compressed-KV rows of a batch of query tokens into a dense bf16 buffer, each
// distinct cache slot once, plus the fan-out table that tells every (token, choice) where its row went.
// Neighbouring query tokens of a prefill chunk select heavily overlapping key sets, so the dense
// buffer is much smaller than tokens x top-k rows and can feed a dense attention GEMM.
//
// Three steps (the prefix sum in the middle is a library scan over the flag array):
//   mark    flags[slot] = 1 for every selected slot
//   (scan)  index[slot] = number of marked slots below it  -> deterministic, ascending-slot order
//   gather  dense[index[slot]] = dequantised row (fp8 latent x group scale | bf16 rope) for marked slots
//   fanout  where[t, j] = index[slots[t, j]]  (-1 for unused entries)
// Reference: `gather_topk_ckv_kernel`, `reset_scratch_kernel`, `mark_unique_kernel`,
// `fanout_topk_ckv_kernel` (`csrc/glm_gather_topk_ckv.cu:97-359`), which claims rows with atomics.
#include "common.cuh"

namespace {

__global__ void mark_slots_kernel(int* __restrict__ flags, const int* __restrict__ slots, const int* __restrict__ lengths, int T, int k) {
    pdl_grid_sync();
    const int t = blockIdx.y;
    const int L = lengths[t];
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < L; j += gridDim.x * blockDim.x) {
        const int s = slots[(size_t)t * k + j];
        if (s >= 0) flags[s] = 1;
    }
}

// One warp per marked slot row.  Row layout: R e4m3 | R/group fp32 scales | Dr bf16.
__global__ void gather_rows_kernel(bf16* __restrict__ dense, const uint8_t* __restrict__ kv_cache, const int* __restrict__ flags,
                                   const int* __restrict__ index, int num_slots, int R, int Dr, int group) {
    pdl_grid_sync();
    const int slot = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (slot >= num_slots || flags[slot] == 0) return;
    const int ngroups = R / group, row_bytes = R + 4 * ngroups + 2 * Dr;
    const uint8_t* row = kv_cache + (size_t)slot * row_bytes;
    bf16* dst = dense + (size_t)index[slot] * (R + Dr);
    for (int d = lane; d < R; d += 32) {
        const float sc = *reinterpret_cast<const float*>(row + R + 4 * (d / group));
        dst[d] = __float2bfloat16(e4m3_to_float(row[d]) * sc);
    }
    const bf16* pe = reinterpret_cast<const bf16*>(row + R + 4 * ngroups);
    for (int d = lane; d < Dr; d += 32) dst[R + d] = pe[d];
}

__global__ void fanout_kernel(int* __restrict__ where, const int* __restrict__ slots, const int* __restrict__ lengths,
                              const int* __restrict__ index, int T, int k) {
    pdl_grid_sync();
    const int t = blockIdx.y;
    const int L = lengths[t];
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < k; j += gridDim.x * blockDim.x) {
        const int s = j < L ? slots[(size_t)t * k + j] : -1;
        where[(size_t)t * k + j] = s >= 0 ? index[s] : -1;
    }
}

}  // namespace

SL_API int sl_gather_mark(void* flags, const void* slots, const void* lengths, int T, int k, cudaStream_t s) {
    if (T == 0) return 0;
    sl_launch(mark_slots_kernel, dim3((k + 255) / 256, T), 256, 0, s, (int*)flags, (const int*)slots, (const int*)lengths, T, k);
    return SL_LAUNCH_CHECK();
}

SL_API int sl_gather_rows(void* dense, const void* kv_cache, const void* flags, const void* index, int num_slots, int R, int Dr,
                          int group, cudaStream_t s) {
    if (num_slots == 0) return 0;
    if (R % group != 0) return -1;
    sl_launch(gather_rows_kernel, (unsigned)(((size_t)num_slots * 32 + 255) / 256), 256, 0, s, (bf16*)dense, (const uint8_t*)kv_cache,
              (const int*)flags, (const int*)index, num_slots, R, Dr, group);
    return SL_LAUNCH_CHECK();
}

SL_API int sl_gather_fanout(void* where, const void* slots, const void* lengths, const void* index, int T, int k, cudaStream_t s) {
    if (T == 0) return 0;
    sl_launch(fanout_kernel, dim3((k + 255) / 256, T), 256, 0, s, (int*)where, (const int*)slots, (const int*)lengths, (const int*)index, T, k);
    return SL_LAUNCH_CHECK();
}
