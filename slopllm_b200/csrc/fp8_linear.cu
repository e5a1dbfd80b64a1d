// Linear layers whose weights stay in FP8 (e4m3 bytes + one fp32 scale per 128 x 128 block, the layout of the
// Qwen3-FP8 checkpoints: `weight` [N, K] and `weight_scale_inv` [ceil(N/128), ceil(K/128)]).
//
//   fp8_gemv_kernel          decode (up to 8 token rows per pass): one warp per output feature streams the weight row
//                            with 16-byte loads, expands e4m3 -> f32 in registers, applies the block scale once per
//                            16-element chunk.  The weights are read once from HBM at one byte per element, which is
//                            the point of keeping them in FP8.
//   fp8_block_dequant_kernel expands a matrix to bf16 for the tensor-core GEMMs (more than 8 rows).
//
// Reference: `fp8_dequantize_gemv_kernel`, `fp8_dequantize_gemm_smem_kernel` (`csrc/glm_gemv.cu:323-500`).
#include "common.cuh"

namespace {

__device__ __forceinline__ void e4m3x16_to_float(const uint4& v, float (&f)[16]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 a = e4m3x2_to_float2((uint16_t)(w[i] & 0xffffu)), b = e4m3x2_to_float2((uint16_t)(w[i] >> 16));
        f[4 * i + 0] = a.x; f[4 * i + 1] = a.y; f[4 * i + 2] = b.x; f[4 * i + 3] = b.y;
    }
}

// grid (ceil(N / 8), ceil(T / TT)), 256 threads: warp w of block b owns output feature 8 b + w for TT token rows.
template <int TT>
__global__ void __launch_bounds__(256) fp8_gemv_kernel(const uint8_t* __restrict__ W, const float* __restrict__ S,
                                                       const bf16* __restrict__ x, void* __restrict__ y, int T, int N, int K,
                                                       int ldx, int ldy, int scale_cols, int out_f32) {
    pdl_grid_sync();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    if (n >= N) return;
    const int t0 = blockIdx.y * TT;
    const uint8_t* wrow = W + (size_t)n * K;
    const float* srow = S + (size_t)(n >> 7) * scale_cols;
    float acc[TT];
#pragma unroll
    for (int t = 0; t < TT; ++t) acc[t] = 0.f;
    for (int k = lane * 16; k < K; k += 32 * 16) {
        float wf[16];
        e4m3x16_to_float(ldg_nc_16(wrow + k), wf);
        const float sc = srow[k >> 7];
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            if (t0 + t < T) {
                const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)(t0 + t) * ldx + k);
                const uint4 x0 = xp[0], x1 = xp[1];
                const uint32_t xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                float d = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float2 xf = bf162_to_f2(xw[i]);
                    d = fmaf(wf[2 * i], xf.x, d);
                    d = fmaf(wf[2 * i + 1], xf.y, d);
                }
                acc[t] = fmaf(sc, d, acc[t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < TT; ++t) {
        const float v = warp_sum(acc[t]);
        if (lane == 0 && t0 + t < T) {
            if (out_f32) ((float*)y)[(size_t)(t0 + t) * ldy + n] = v;
            else ((bf16*)y)[(size_t)(t0 + t) * ldy + n] = __float2bfloat16(v);
        }
    }
}

// One thread per 16 consecutive elements of a row.
__global__ void fp8_block_dequant_kernel(bf16* __restrict__ out, const uint8_t* __restrict__ W, const float* __restrict__ S, int N,
                                         int K, int scale_cols) {
    pdl_grid_sync();
    const int units = K / 16;
    const size_t total = (size_t)N * units;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int n = (int)(i / units), k = (int)(i % units) * 16;
        float wf[16];
        e4m3x16_to_float(ldg_nc_16(W + (size_t)n * K + k), wf);
        const float sc = S[(size_t)(n >> 7) * scale_cols + (k >> 7)];
        uint4 o0, o1;
        o0.x = f2_to_bf162(wf[0] * sc, wf[1] * sc);   o0.y = f2_to_bf162(wf[2] * sc, wf[3] * sc);
        o0.z = f2_to_bf162(wf[4] * sc, wf[5] * sc);   o0.w = f2_to_bf162(wf[6] * sc, wf[7] * sc);
        o1.x = f2_to_bf162(wf[8] * sc, wf[9] * sc);   o1.y = f2_to_bf162(wf[10] * sc, wf[11] * sc);
        o1.z = f2_to_bf162(wf[12] * sc, wf[13] * sc); o1.w = f2_to_bf162(wf[14] * sc, wf[15] * sc);
        uint4* dst = reinterpret_cast<uint4*>(out + (size_t)n * K + k);
        dst[0] = o0;
        dst[1] = o1;
    }
}

}  // namespace

// y[T, N] = x[T, K] (bf16, row stride ldx) * dequant(W)^T, W [N, K] e4m3 bytes (contiguous), S [ceil(N/128), scale_cols] fp32
// with scale_cols >= ceil(K/128).  K % 16 == 0, ldx % 8 == 0, W 16-byte aligned.  T <= 32 (token rows go in passes of up to 8,
// each of which streams the weights again).
SL_API int sl_linear_fp8_block(const void* x, const void* W, const void* S, void* y, int T, int N, int K, int ldx, int ldy,
                               int scale_cols, int out_f32, cudaStream_t s) {
    if (T <= 0 || N <= 0 || K <= 0) return 0;
    if (T > 32 || K % 16 != 0 || ldx % 8 != 0 || scale_cols < (K + 127) / 128 || ((uintptr_t)W & 15) != 0 || ((uintptr_t)x & 15) != 0)
        return -1;
    const int tt = T == 1 ? 1 : (T == 2 ? 2 : (T <= 4 ? 4 : 8));
    dim3 grid((N + 7) / 8, (T + tt - 1) / tt);
    const uint8_t* w8 = (const uint8_t*)W;
    const float* sc = (const float*)S;
    const bf16* xb = (const bf16*)x;
    if (tt == 1) sl_launch(fp8_gemv_kernel<1>, grid, 256, 0, s, w8, sc, xb, y, T, N, K, ldx, ldy, scale_cols, out_f32);
    else if (tt == 2) sl_launch(fp8_gemv_kernel<2>, grid, 256, 0, s, w8, sc, xb, y, T, N, K, ldx, ldy, scale_cols, out_f32);
    else if (tt == 4) sl_launch(fp8_gemv_kernel<4>, grid, 256, 0, s, w8, sc, xb, y, T, N, K, ldx, ldy, scale_cols, out_f32);
    else sl_launch(fp8_gemv_kernel<8>, grid, 256, 0, s, w8, sc, xb, y, T, N, K, ldx, ldy, scale_cols, out_f32);
    return SL_LAUNCH_CHECK();
}

// out [N, K] bf16 (contiguous) = dequant(W).  K % 16 == 0.
SL_API int sl_fp8_block_dequant_bf16(void* out, const void* W, const void* S, int N, int K, int scale_cols, cudaStream_t s) {
    if (N <= 0 || K <= 0) return 0;
    if (K % 16 != 0 || scale_cols < (K + 127) / 128 || ((uintptr_t)W & 15) != 0 || ((uintptr_t)out & 15) != 0) return -1;
    const size_t total = (size_t)N * (K / 16);
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    sl_launch(fp8_block_dequant_kernel, blocks, 256, 0, s, (bf16*)out, (const uint8_t*)W, (const float*)S, N, K, scale_cols);
    return SL_LAUNCH_CHECK();
}
