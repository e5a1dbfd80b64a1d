// FP8 activation quantisation and an L2 prefetch helper (sm_100a).
//
//  * quantize_fp8_kernel: e4m3 values with one power-of-two fp32 scale per 128-value block of the last
//    dimension (scale = 2^ceil(log2(amax / 448))), the activation format of the FP8 block-scaled linears.
//    Reference: `quantize_fp8_kernel` (`csrc/glm_quantize.cu:1-73`).
//  * prefetch_l2_kernel: `prefetch.global.L2` over a byte range, launched on a side stream to pull the next
//    layer's weights into the 126 MB L2 while the current layer computes (reference `prefetch_l2`,
//    `csrc/glm_ops.cu`).
#include "common.cuh"

namespace {

// One warp per 128-value block: 4 values per lane.
__global__ void quantize_fp8_kernel(uint8_t* __restrict__ q, float* __restrict__ scales, const bf16* __restrict__ x, size_t blocks,
                                    int blocks_per_row, int K) {
    pdl_grid_sync();
    const size_t b = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (b >= blocks) return;
    const size_t row = b / blocks_per_row;
    const int kb = (int)(b % blocks_per_row) * 128;
    const bf16* src = x + row * K + kb;
    float v[4];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int k = lane * 4 + i;
        v[i] = kb + k < K ? __bfloat162float(src[k]) : 0.f;
        amax = fmaxf(amax, fabsf(v[i]));
    }
    amax = warp_max(amax);
    const float scale = pow2_scale_ceil(amax);
    if (lane == 0) scales[b] = scale;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int k = lane * 4 + i;
        if (kb + k < K) q[row * K + kb + k] = float_to_e4m3(v[i] / scale);
    }
}

__global__ void prefetch_l2_kernel(const uint8_t* __restrict__ p, size_t nbytes) {
    pdl_grid_sync();
    for (size_t off = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 128; off < nbytes; off += (size_t)gridDim.x * blockDim.x * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p + off));
}

constexpr int kPrefetchRanges = 12;
struct PrefetchList {
    const uint8_t* ptr[kPrefetchRanges];
    unsigned long long lines[kPrefetchRanges];      // 128-byte lines of each range
    int count;
    int keep;                                       // 1: mark the lines evict-last (streaming traffic passes them by)
};

// One launch for several weight tensors of the next layer: the lines of all ranges are numbered consecutively and
// spread over the grid.
__global__ void prefetch_l2_multi_kernel(PrefetchList l) {
    pdl_grid_sync();
    unsigned long long total = 0;
    for (int i = 0; i < l.count; ++i) total += l.lines[i];
    for (unsigned long long n = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; n < total;
         n += (unsigned long long)gridDim.x * blockDim.x) {
        unsigned long long k = n;
        int i = 0;
        while (k >= l.lines[i]) { k -= l.lines[i]; ++i; }
        const uint8_t* a = l.ptr[i] + k * 128;
        if (l.keep) asm volatile("prefetch.global.L2::evict_last [%0];" ::"l"(a));
        else asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
    }
}

}  // namespace

// Up to 12 byte ranges in one launch (`ptr[i]`, `bytes[i]`); `keep` marks the lines evict-last.
SL_API int sl_prefetch_l2_multi(const void* const* ptrs, const unsigned long long* bytes, int count, int keep, cudaStream_t s) {
    if (count <= 0) return 0;
    if (count > kPrefetchRanges) return -1;
    PrefetchList l{};
    unsigned long long total = 0;
    for (int i = 0; i < count; ++i) {
        l.ptr[i] = (const uint8_t*)ptrs[i];
        l.lines[i] = (bytes[i] + 127) / 128;
        total += l.lines[i];
    }
    l.count = count;
    l.keep = keep;
    if (total == 0) return 0;
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (blocks > 148 * 2) blocks = 148 * 2;
    sl_launch(prefetch_l2_multi_kernel, blocks, 256, 0, s, l);
    return SL_LAUNCH_CHECK();
}

// x [rows, K] bf16 -> q [rows, K] e4m3 bytes, scales [rows, ceil(K / 128)] fp32.
SL_API int sl_quantize_fp8(void* q, void* scales, const void* x, int rows, int K, cudaStream_t s) {
    if (rows == 0 || K == 0) return 0;
    const int bpr = (K + 127) / 128;
    const size_t blocks = (size_t)rows * bpr;
    sl_launch(quantize_fp8_kernel, (unsigned)((blocks * 32 + 255) / 256), 256, 0, s, (uint8_t*)q, (float*)scales, (const bf16*)x, blocks,
              bpr, K);
    return SL_LAUNCH_CHECK();
}

SL_API int sl_prefetch_l2(const void* p, size_t nbytes, cudaStream_t s) {
    if (nbytes == 0) return 0;
    size_t lines = (nbytes + 127) / 128;
    unsigned blocks = (unsigned)((lines + 255) / 256);
    if (blocks > 148 * 4) blocks = 148 * 4;
    sl_launch(prefetch_l2_kernel, blocks, 256, 0, s, (const uint8_t*)p, nbytes);
    return SL_LAUNCH_CHECK();
}
