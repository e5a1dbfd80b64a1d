// Stable counting sort of MoE routes by expert for the prefill path: route r = token * k + j goes to expert ids[r];
// the sorted order groups the rows of each local expert (experts outside [expert_offset, expert_offset + E) sort to
// the end) and keeps routes of one expert in route order, so the result is the same on every run.
// Three small launches replace a radix sort + histogram + scan sequence (reference: `histogram_kernel` /
// `prefix_sum_kernel` / `scatter_input_kernel`, `csrc/glm_mma_moe.cu:387-460`).
#include "common.cuh"

namespace {

constexpr int SORT_BLOCK = 1024;

__device__ __forceinline__ int route_key(const int* ids, int r, int n, int expert_offset, int E) {
    if (r >= n) return -1;
    const int e = ids[r] - expert_offset;
    return (e >= 0 && e < E) ? e : E;
}

// block_hist[b][e] = routes of block b with key e (e == E: not local)
__global__ void __launch_bounds__(SORT_BLOCK) moe_sort_count_kernel(const int* __restrict__ ids, int n, int expert_offset, int E,
                                                                    int* __restrict__ block_hist) {
    pdl_grid_sync();
    extern __shared__ int hist[];                       // E + 1
    for (int i = threadIdx.x; i <= E; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const int key = route_key(ids, blockIdx.x * SORT_BLOCK + threadIdx.x, n, expert_offset, E);
    if (key >= 0) atomicAdd(&hist[key], 1);
    __syncthreads();
    for (int i = threadIdx.x; i <= E; i += blockDim.x) block_hist[(size_t)blockIdx.x * (E + 1) + i] = hist[i];
}

// offsets[e] = first sorted row of key e (offsets[E] = number of local rows); block_hist[b][e] becomes the first sorted row
// of block b's routes with key e.  One block of 1024 threads, E + 1 <= 1024.
__global__ void __launch_bounds__(1024) moe_sort_scan_kernel(int* __restrict__ block_hist, int blocks, int E, int* __restrict__ offsets) {
    pdl_grid_sync();
    __shared__ int total[1024];
    __shared__ int base[1025];
    const int e = threadIdx.x;
    int sum = 0;
    if (e <= E)
        for (int b = 0; b < blocks; ++b) sum += block_hist[(size_t)b * (E + 1) + e];
    total[e] = e <= E ? sum : 0;
    __syncthreads();
    if (e == 0) {
        int run = 0;
        for (int i = 0; i <= E; ++i) { base[i] = run; run += total[i]; }
        base[E + 1] = run;
    }
    __syncthreads();
    if (e <= E) {
        offsets[e] = base[e];
        int run = base[e];
        for (int b = 0; b < blocks; ++b) {
            const int c = block_hist[(size_t)b * (E + 1) + e];
            block_hist[(size_t)b * (E + 1) + e] = run;
            run += c;
        }
    }
}

// order[pos] = route, src_tok[pos] = route / k, rows_of[route] = pos (or -1 when the expert is not local)
__global__ void __launch_bounds__(SORT_BLOCK) moe_sort_scatter_kernel(const int* __restrict__ ids, int n, int k, int expert_offset, int E,
                                                                      const int* __restrict__ block_off, int* __restrict__ order,
                                                                      int* __restrict__ rows_of, int* __restrict__ src_tok) {
    pdl_grid_sync();
    extern __shared__ int cnt[];                        // [32 warps][E + 1]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, W = E + 1;
    for (int i = threadIdx.x; i < 32 * W; i += blockDim.x) cnt[i] = 0;
    __syncthreads();
    const int r = blockIdx.x * SORT_BLOCK + threadIdx.x;
    const int key = route_key(ids, r, n, expert_offset, E);
    const unsigned same = __match_any_sync(0xffffffffu, key);
    const int rank_in_warp = __popc(same & ((1u << lane) - 1u));
    if (key >= 0 && rank_in_warp == 0) cnt[warp * W + key] = __popc(same);
    __syncthreads();
    // exclusive prefix over the warps, per key
    for (int e = threadIdx.x; e < W; e += blockDim.x) {
        int run = 0;
        for (int w = 0; w < 32; ++w) {
            const int c = cnt[w * W + e];
            cnt[w * W + e] = run;
            run += c;
        }
    }
    __syncthreads();
    if (key >= 0) {
        const int pos = block_off[(size_t)blockIdx.x * W + key] + cnt[warp * W + key] + rank_in_warp;
        order[pos] = r;
        src_tok[pos] = r / k;
        rows_of[r] = key < E ? pos : -1;
    }
}

}  // namespace

// ids [n] int32 (n = tokens * k routes).  scratch: at least ceil(n / 1024) * (E + 1) ints.  Outputs: offsets [E + 1],
// order [n], rows_of [n], src_tok [n] (all int32).  E + 1 <= 1024.
SL_API int sl_moe_sort_routes(const void* ids, int n, int k, int expert_offset, int E, void* scratch, void* offsets, void* order,
                              void* rows_of, void* src_tok, cudaStream_t s) {
    if (n <= 0) return 0;
    if (E <= 0 || E + 1 > 1024 || k <= 0) return -1;
    const int blocks = (n + SORT_BLOCK - 1) / SORT_BLOCK;
    const size_t sm_hist = (size_t)(E + 1) * sizeof(int), sm_cnt = (size_t)32 * (E + 1) * sizeof(int);
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(moe_sort_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * 1024 * (int)sizeof(int));
        attr = true;
    }
    sl_launch(moe_sort_count_kernel, blocks, SORT_BLOCK, sm_hist, s, (const int*)ids, n, expert_offset, E, (int*)scratch);
    sl_launch(moe_sort_scan_kernel, 1, 1024, 0, s, (int*)scratch, blocks, E, (int*)offsets);
    sl_launch(moe_sort_scatter_kernel, blocks, SORT_BLOCK, sm_cnt, s, (const int*)ids, n, k, expert_offset, E, (const int*)scratch,
              (int*)order, (int*)rows_of, (int*)src_tok);
    return (int)cudaGetLastError();
}
