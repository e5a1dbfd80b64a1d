// Vocabulary arg-max that brings its own scratch memory (see no_alloc.h for who needs this and
// the rules of use).  Two stages like sl_argmax: 64 partial winners per row, then one warp per
// row; the partials live in the file-scope array below rather than in caller-provided memory.
#include <cstdio>

#include "common.cuh"
#include "no_alloc.h"

namespace {

constexpr int kChunks = 64;
constexpr int kMaxDevices = 64;

struct Partial {
    float value;
    int index;
};

// 256 rows x 64 chunks x 8 bytes = 128 KiB, resident on every device that loads the library.
static __device__ __align__(256) Partial g_scratch[SL_ARGMAX_NOALLOC_MAX_ROWS * kChunks];

// Device address of g_scratch per device ordinal, resolved on first use.  In host code the name
// `g_scratch` is only a handle for the runtime, never an address a kernel may dereference.
Partial* g_scratch_addr[kMaxDevices] = {};

template <typename TL>
__global__ void __launch_bounds__(256) partial_kernel(Partial* __restrict__ part, const TL* __restrict__ logits, int V, int ld) {
    __shared__ float sv[8];
    __shared__ int si[8];
    const int b = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per = (V + gridDim.x - 1) / gridDim.x;
    const int lo = blockIdx.x * per, hi = min(V, lo + per);
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = (float)logits[(size_t)b * ld + i];
        if (v > best) { best = v; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
        part[(size_t)b * gridDim.x + blockIdx.x] = Partial{best, bi};      // every slot read later is written here
    }
}

__global__ void final_kernel(int64_t* __restrict__ out, float* __restrict__ out_val, const Partial* __restrict__ part,
                             int chunks, int64_t id_offset) {
    const int b = blockIdx.x, lane = threadIdx.x;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lane; i < chunks; i += 32) {
        const Partial p = part[(size_t)b * chunks + i];
        if (p.value > best || (p.value == best && p.index < bi)) { best = p.value; bi = p.index; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) {
        if (bi == 0x7fffffff) bi = 0;
        out[b] = (int64_t)bi + id_offset;
        if (out_val) out_val[b] = best;
    }
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int sl_argmax_noalloc(void* out_ids, const void* logits, int rows, int vocab,
                                                                         int ld, int logits_are_f32, long long id_offset,
                                                                         void* out_values, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (out_ids == nullptr || logits == nullptr || rows < 0 || vocab <= 0 || ld < vocab) {
        fprintf(stderr, "sl_argmax_noalloc: bad argument (rows=%d vocab=%d ld=%d)\n", rows, vocab, ld);
        return SL_NOALLOC_E_BAD_ARG;
    }
    if (rows > SL_ARGMAX_NOALLOC_MAX_ROWS) {
        fprintf(stderr, "sl_argmax_noalloc: %d rows exceed the built-in scratch (max %d rows); split the batch or use sl_argmax\n",
                rows, SL_ARGMAX_NOALLOC_MAX_ROWS);
        return SL_NOALLOC_E_TOO_LARGE;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return SL_NOALLOC_E_SETUP;
    if (g_scratch_addr[dev] == nullptr) {
        // once per device, with that device current: resolve the device address of the array
        Partial* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_scratch);
        if (e != cudaSuccess || p == nullptr) {
            fprintf(stderr, "sl_argmax_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev, cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : SL_NOALLOC_E_SETUP;
        }
        g_scratch_addr[dev] = p;
    }
    Partial* scratch = g_scratch_addr[dev];
    dim3 grid(kChunks, rows);
    if (logits_are_f32) partial_kernel<float><<<grid, 256, 0, stream>>>(scratch, (const float*)logits, vocab, ld);
    else partial_kernel<bf16><<<grid, 256, 0, stream>>>(scratch, (const bf16*)logits, vocab, ld);
    final_kernel<<<rows, 32, 0, stream>>>((int64_t*)out_ids, (float*)out_values, scratch, kChunks, id_offset);
    return (int)cudaGetLastError();
}
