// NVFP4 weights x a few activation rows (2..32 tokens: batched decode, MTP verification):
// the packed weights are streamed from HBM once, expanded E2M1 -> f16 (x UE4M3 block scale) in
// registers and fed to the tensor cores as the 16-row operand of `mma.sync.m16n8k16`; the
// tokens are the 8-wide operand.  W4A16: activations stay f16.
//
// Work split: a warp owns 16 (or 32) output features and every ksplit-th group of 128 reduction
// indices, so that one 16-byte load per lane covers a row's 32 consecutive codes; the warps of
// a block that share rows meet in shared memory at the end.  The reduction index is consumed
// in a permuted order (a lane's 32 codes feed 8 MMAs, 4 codes each); a small kernel first
// writes the activations as f16 in exactly that order, so that each lane's operand is one
// 16-byte L1-cached load.
//
// Reference counterpart: `nvfp4_dequantize_gemm_smem_kernel` (`csrc/glm_gemv.cu:653`, batch 3-16
// on CUDA cores) and the MoE small-batch kernels (`:738-990`).
#include "push.cuh"

namespace {

__device__ __forceinline__ void mma_f16_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ __half2 e4m3x2_to_half2(uint16_t v) {
    __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)v, __NV_E4M3);
    return *reinterpret_cast<__half2*>(&h);
}

// ---- activation staging --------------------------------------------------------------------------
// x[T, K] bf16 -> f16 in fragment order in global scratch: 16-byte unit(token, group, j, c) holds
// x[token][group*128 + c*32 + j*8 .. +7] at unit index (token*G + group)*16 + j*4 + c, G = K/128.
// Rows T..tpad-1 are zero.
__global__ void permute_x_kernel(uint4* __restrict__ xp, const bf16* __restrict__ x, int T, int tpad, int K, int ldx) {
    const int units = tpad * (K / 8);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < units; i += gridDim.x * blockDim.x) {
        const int tok = i / (K / 8), u = i % (K / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tok < T) {
            const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)tok * ldx + u * 8);
            const float2 f0 = bf162_to_f2(raw.x), f1 = bf162_to_f2(raw.y), f2 = bf162_to_f2(raw.z), f3 = bf162_to_f2(raw.w);
            __half2 h0 = __floats2half2_rn(f0.x, f0.y), h1 = __floats2half2_rn(f1.x, f1.y);
            __half2 h2 = __floats2half2_rn(f2.x, f2.y), h3 = __floats2half2_rn(f3.x, f3.y);
            v.x = *reinterpret_cast<uint32_t*>(&h0); v.y = *reinterpret_cast<uint32_t*>(&h1);
            v.z = *reinterpret_cast<uint32_t*>(&h2); v.w = *reinterpret_cast<uint32_t*>(&h3);
        }
        const int group = u / 16, within = u % 16, c = within / 4, j = within % 4;
        xp[((size_t)tok * (K / 128) + group) * 16 + j * 4 + c] = v;
    }
}

// Expand one lane's 16 bytes (32 codes) of a row into 16 half2, scaled by the two block scales.
__device__ __forceinline__ void expand_row(const uint4& w, uint16_t sc, __half2 (&out)[16]) {
    const __half2 s = e4m3x2_to_half2(sc);
    const __half2 s0 = __half2half2(__low2half(s)), s1 = __half2half2(__high2half(s));
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        __half2 h[4];
        e2m1x8_to_half2x4(words[q], h);
        const __half2 sq = q < 2 ? s0 : s1;
#pragma unroll
        for (int i = 0; i < 4; ++i) out[q * 4 + i] = __hmul2(h[i], sq);
    }
}

__device__ __forceinline__ uint4 ldg_ca_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// One warp: MT tiles of 16 rows x NT*8 tokens over the groups kpart, kpart+ksplit, ... of the row's K.
template <int MT, int NT>
__device__ __forceinline__ void warp_rows_times_tokens(float (&acc)[MT][NT][4], const uint8_t* __restrict__ Wp,
                                                       const uint8_t* __restrict__ S, size_t w_stride, size_t s_stride,
                                                       int rows_valid, int K, const uint4* __restrict__ xp, int kpart, int ksplit) {
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int G = K / 128;
    // software pipeline: raw rows of the next group are in flight while this group is expanded
    uint4 w0[MT], w1[MT], w0n[MT], w1n[MT];
    uint16_t s0[MT], s1[MT], s0n[MT], s1n[MT];
    auto load_group = [&](int group, uint4 (&a0)[MT], uint4 (&a1)[MT], uint16_t (&b0)[MT], uint16_t (&b1)[MT]) {
        const int kk = group * 128 + c * 32;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            a0[mt] = make_uint4(0, 0, 0, 0); a1[mt] = a0[mt]; b0[mt] = 0; b1[mt] = 0;
            const int ra = mt * 16 + g, rb = ra + 8;
            if (group < G && ra < rows_valid) {
                a0[mt] = ldg_nc_16(Wp + (size_t)ra * w_stride + (kk >> 1));
                b0[mt] = *reinterpret_cast<const uint16_t*>(S + (size_t)ra * s_stride + (kk >> 4));
            }
            if (group < G && rb < rows_valid) {
                a1[mt] = ldg_nc_16(Wp + (size_t)rb * w_stride + (kk >> 1));
                b1[mt] = *reinterpret_cast<const uint16_t*>(S + (size_t)rb * s_stride + (kk >> 4));
            }
        }
    };
    load_group(kpart, w0, w1, s0, s1);
    for (int group = kpart; group < G; group += ksplit) {
        load_group(group + ksplit, w0n, w1n, s0n, s1n);
        __half2 a_lo[MT][16], a_hi[MT][16];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            expand_row(w0[mt], s0[mt], a_lo[mt]);
            expand_row(w1[mt], s1[mt], a_hi[mt]);
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint4* xr = xp + ((size_t)(nt * 8 + g) * G + group) * 16 + c;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 xv = ldg_ca_16(xr + j * 4);          // x[token][kk + j*8 .. +7]
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    // codes 8j..8j+3 -> first MMA ; codes 8j+4..8j+7 -> second MMA
                    uint32_t a[4];
                    a[0] = *reinterpret_cast<const uint32_t*>(&a_lo[mt][4 * j + 0]);
                    a[1] = *reinterpret_cast<const uint32_t*>(&a_hi[mt][4 * j + 0]);
                    a[2] = *reinterpret_cast<const uint32_t*>(&a_lo[mt][4 * j + 1]);
                    a[3] = *reinterpret_cast<const uint32_t*>(&a_hi[mt][4 * j + 1]);
                    mma_f16_m16n8k16(acc[mt][nt], a, xv.x, xv.y);
                    a[0] = *reinterpret_cast<const uint32_t*>(&a_lo[mt][4 * j + 2]);
                    a[1] = *reinterpret_cast<const uint32_t*>(&a_hi[mt][4 * j + 2]);
                    a[2] = *reinterpret_cast<const uint32_t*>(&a_lo[mt][4 * j + 3]);
                    a[3] = *reinterpret_cast<const uint32_t*>(&a_hi[mt][4 * j + 3]);
                    mma_f16_m16n8k16(acc[mt][nt], a, xv.z, xv.w);
                }
            }
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) { w0[mt] = w0n[mt]; w1[mt] = w1n[mt]; s0[mt] = s0n[mt]; s1[mt] = s1n[mt]; }
    }
}

// Block = 8 warps = (8 / ksplit) row tiles x ksplit reduction parts; a row tile is MT*16 features.
// Partial tiles meet in shared memory: red[warp][token][MT*16].
template <int MT, int NT>
__global__ void __launch_bounds__(256) linear_nvfp4_mma_kernel(void* __restrict__ y, const uint4* __restrict__ xp,
                                                               const uint8_t* __restrict__ Wp, const uint8_t* __restrict__ S,
                                                               const float* __restrict__ gscale, int T, int N, int K,
                                                               int ksplit, int out_f32, int use_push, PushCtx push) {
    extern __shared__ float red[];
    constexpr int ROWS = MT * 16, TOK = NT * 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int tiles_per_block = 8 / ksplit;
    const int tile = warp / ksplit, kpart = warp % ksplit;
    const int n0 = (blockIdx.x * tiles_per_block + tile) * ROWS;
    float acc[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.f;
    if (n0 < N)
        warp_rows_times_tokens<MT, NT>(acc, Wp + (size_t)n0 * (K / 2), S + (size_t)n0 * (K / 16), K / 2, K / 16, min(ROWS, N - n0), K,
                                       xp, kpart, ksplit);
    float* mine = red + (size_t)warp * (TOK * ROWS);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            // d0:(row g, tok 2c) d1:(row g, tok 2c+1) d2:(row g+8, tok 2c) d3:(row g+8, tok 2c+1)
            mine[(nt * 8 + 2 * c) * ROWS + mt * 16 + g] = acc[mt][nt][0];
            mine[(nt * 8 + 2 * c + 1) * ROWS + mt * 16 + g] = acc[mt][nt][1];
            mine[(nt * 8 + 2 * c) * ROWS + mt * 16 + g + 8] = acc[mt][nt][2];
            mine[(nt * 8 + 2 * c + 1) * ROWS + mt * 16 + g + 8] = acc[mt][nt][3];
        }
    __syncthreads();
    const float gs = gscale ? *gscale : 1.f;
    for (int i = threadIdx.x; i < tiles_per_block * TOK * ROWS; i += blockDim.x) {
        const int tl = i / (TOK * ROWS), rem = i % (TOK * ROWS), tok = rem / ROWS, r = rem % ROWS;
        const int n = (blockIdx.x * tiles_per_block + tl) * ROWS + r;
        if (tok < T && n < N) {
            float v = 0.f;
            for (int kp = 0; kp < ksplit; ++kp) v += red[(size_t)(tl * ksplit + kp) * (TOK * ROWS) + rem];
            v *= gs;
            if (use_push) {
                // fused all-reduce, producer side: the partial goes to every rank's receive slot
                for (int pr = 0; pr < push.world; ++pr) *push_dst(push, pr, tok, n) = v;
            } else if (out_f32) ((float*)y)[(size_t)tok * N + n] = v;
            else ((bf16*)y)[(size_t)tok * N + n] = __float2bfloat16(v);
        }
    }
    if (use_push) push_finish(push, gridDim.x);
}

template <int MT, int NT>
int launch_linear(void* y, const void* x, void* xp, const void* Wp, const void* S, const void* g, int T, int N, int K, int ldx,
                  int out_f32, const PushCtx* push, cudaStream_t s) {
    constexpr int ROWS = MT * 16, TOK = NT * 8;
    const int units = TOK * (K / 8);
    permute_x_kernel<<<(units + 255) / 256, 256, 0, s>>>((uint4*)xp, (const bf16*)x, T, TOK, K, ldx);
    int ksplit = 8;
    while (ksplit > 1 && K / 128 < ksplit) ksplit >>= 1;
    // few rows: keep the reduction split so that there are enough blocks to fill the machine
    const int tiles = (N + ROWS - 1) / ROWS;
    const int tiles_per_block = 8 / ksplit;
    auto kern = linear_nvfp4_mma_kernel<MT, NT>;
    const size_t smem = (size_t)8 * TOK * ROWS * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<(tiles + tiles_per_block - 1) / tiles_per_block, 256, smem, s>>>(y, (const uint4*)xp, (const uint8_t*)Wp,
                                                                           (const uint8_t*)S, (const float*)g, T, N, K, ksplit,
                                                                           out_f32, push ? 1 : 0, push ? *push : PushCtx{});
    return (int)cudaGetLastError();
}

}  // namespace

static int dispatch_linear(void* y, const void* x, void* xp, const void* Wp, const void* S, const void* g, int T, int N, int K,
                           int ldx, int out_f32, const PushCtx* push, cudaStream_t s) {
    if (T == 0 || N == 0) return 0;
    if (T > 32 || K % 128 != 0 || ldx % 8 != 0) return -1;
    if (T <= 8) return launch_linear<1, 1>(y, x, xp, Wp, S, g, T, N, K, ldx, out_f32, push, s);
    if (T <= 16) return launch_linear<1, 2>(y, x, xp, Wp, S, g, T, N, K, ldx, out_f32, push, s);
    if (T <= 24) return launch_linear<2, 3>(y, x, xp, Wp, S, g, T, N, K, ldx, out_f32, push, s);
    return launch_linear<2, 4>(y, x, xp, Wp, S, g, T, N, K, ldx, out_f32, push, s);
}

// y[T, N] = g * x[T, K] . dequant(Wp, S)^T for 1 <= T <= 32.  K % 128 == 0, ldx % 8 == 0.
// `xp` is caller-owned scratch of ceil(T/8)*8 * K f16 values (the permuted copy of x).
SL_API int sl_linear_nvfp4_mma(void* y, const void* x, void* xp, const void* Wp, const void* S, const void* g, int T, int N,
                               int K, int ldx, int out_f32, cudaStream_t s) {
    return dispatch_linear(y, x, xp, Wp, S, g, T, N, K, ldx, out_f32, nullptr, s);
}

// Same product, but the fp32 result rows are stored into every rank's receive slot and the epoch
// flags are published (producer half of the fused all-reduce; consumer: sl_ar_add_rmsnorm).
SL_API int sl_linear_nvfp4_mma_push(const void* x, void* xp, const void* Wp, const void* S, const void* g, int T, int N, int K,
                                    int ldx, const PushCtx* push, cudaStream_t s) {
    if (push == nullptr || T > push->slot_rows || N > push->row_len) return -1;
    return dispatch_linear(nullptr, x, xp, Wp, S, g, T, N, K, ldx, 1, push, s);
}
