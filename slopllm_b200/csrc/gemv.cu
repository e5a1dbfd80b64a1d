// Small-batch (decode) linear layers: weights are streamed from HBM exactly once per
// step, activations (<= 32 token rows) live in shared memory.  bf16 and NVFP4
// (E2M1 x UE4M3 block scale x f32 global) weights; dense and per-route (MoE) forms.
//
// Reference counterparts: `csrc/glm_gemv.cu:80-320` (bf16 GEMV), `:505-735` (NVFP4 GEMV),
// `:738-990` (nvfp4_mul_mat_id), `:1291-1375` (fused down-proj + weighted top-k reduce).
// The kernels here are memory-roofline designs for HBM3e: 16-byte non-allocating loads,
// several rows in flight per warp, fp32 accumulation.
#include "push.cuh"

// ---------------------------------------------------------------------------------------------
// bf16: y[t, n] = sum_k x[t, k] W[n, k].   Warp handles R rows at a time for TT tokens.
template <int TT, int R>
__global__ void __launch_bounds__(256) gemv_bf16_kernel(void* __restrict__ y, const bf16* __restrict__ x,
                                                        const bf16* __restrict__ W, int T, int N, int K, int ldx,
                                                        int out_f32, const float* __restrict__ bias) {
    // first rows of every warp of this block: 8 warps x R rows, whole rows
    PDL_ENTRY_WITH_PREFETCH({
        const int first = blockIdx.x * 8 * R;
        if (first < N) prefetch_l2_rows(W + (size_t)first * K, min(8 * R, N - first), (size_t)K * 2);
    });
    extern __shared__ __align__(16) unsigned char smraw[];
    bf16* xs = reinterpret_cast<bf16*>(smraw);           // [TT][K]
    const int t0 = blockIdx.y * TT;
    for (int i = threadIdx.x; i < TT * (K / 8); i += blockDim.x) {
        const int tt = i / (K / 8), c = i % (K / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t0 + tt < T) v = *reinterpret_cast<const uint4*>(x + (size_t)(t0 + tt) * ldx + c * 8);
        reinterpret_cast<uint4*>(xs)[i] = v;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
    for (int n0 = warp * R; n0 < N; n0 += nwarps * R) {
        float acc[R][TT];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) acc[r][tt] = 0.f;
        // U chunks of 256 reduction indices per step, every load of the step issued before the first use
        constexpr int U = (R * TT <= 4) ? 4 : 2;
        for (int k0 = lane * 8; k0 < K; k0 += 256 * U) {
            uint4 w[U][R];
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int k = k0 + u * 256;
                    w[u][r] = (k < K && n0 + r < N) ? ldg_nc_16(W + (size_t)(n0 + r) * K + k) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int k = k0 + u * 256;
                if (k >= K) break;
#pragma unroll
                for (int tt = 0; tt < TT; ++tt) {
                    const uint4 xv = *reinterpret_cast<const uint4*>(xs + tt * K + k);
                    const float2 x0 = bf162_to_f2(xv.x), x1 = bf162_to_f2(xv.y), x2 = bf162_to_f2(xv.z), x3 = bf162_to_f2(xv.w);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const float2 w0 = bf162_to_f2(w[u][r].x), w1 = bf162_to_f2(w[u][r].y), w2 = bf162_to_f2(w[u][r].z),
                                     w3 = bf162_to_f2(w[u][r].w);
                        acc[r][tt] += x0.x * w0.x + x0.y * w0.y + x1.x * w1.x + x1.y * w1.y + x2.x * w2.x + x2.y * w2.y +
                                      x3.x * w3.x + x3.y * w3.y;
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) {
                const float v = warp_sum(acc[r][tt]);
                if (lane == 0 && n0 + r < N && t0 + tt < T) {
                    const float o = v + (bias ? bias[n0 + r] : 0.f);
                    if (out_f32) ((float*)y)[(size_t)(t0 + tt) * N + n0 + r] = o;
                    else ((bf16*)y)[(size_t)(t0 + tt) * N + n0 + r] = __float2bfloat16(o);
                }
            }
    }
    pdl_trigger_late();
}

// Small N (router, narrow projections): one block per output row, the 256 threads split K.
template <int TT>
__global__ void __launch_bounds__(256) gemv_bf16_rowblock_kernel(void* __restrict__ y, const bf16* __restrict__ x,
                                                                 const bf16* __restrict__ W, int T, int N, int K, int ldx,
                                                                 int out_f32) {
    pdl_grid_sync();
    __shared__ float scratch[33];
    const int n = blockIdx.x, t0 = blockIdx.y * TT;
    float acc[TT];
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) acc[tt] = 0.f;
    for (int k = threadIdx.x * 8; k < K; k += 256 * 8) {
        const uint4 w = ldg_nc_16(W + (size_t)n * K + k);
        const float2 w0 = bf162_to_f2(w.x), w1 = bf162_to_f2(w.y), w2 = bf162_to_f2(w.z), w3 = bf162_to_f2(w.w);
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
            if (t0 + tt < T) {
                const uint4 xv = *reinterpret_cast<const uint4*>(x + (size_t)(t0 + tt) * ldx + k);
                const float2 x0 = bf162_to_f2(xv.x), x1 = bf162_to_f2(xv.y), x2 = bf162_to_f2(xv.z), x3 = bf162_to_f2(xv.w);
                acc[tt] += x0.x * w0.x + x0.y * w0.y + x1.x * w1.x + x1.y * w1.y + x2.x * w2.x + x2.y * w2.y + x3.x * w3.x +
                           x3.y * w3.y;
            }
        }
    }
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
        const float v = block_sum(acc[tt], scratch);
        if (threadIdx.x == 0 && t0 + tt < T) {
            if (out_f32) ((float*)y)[(size_t)(t0 + tt) * N + n] = v;
            else ((bf16*)y)[(size_t)(t0 + tt) * N + n] = __float2bfloat16(v);
        }
    }
}

template <int TT, int R>
static int launch_gemv_bf16_r(void* y, const void* x, const void* W, int T, int N, int K, int ldx, int out_f32, cudaStream_t s) {
    const size_t smem = (size_t)TT * K * sizeof(bf16);
    const int tiles = (T + TT - 1) / TT;
    auto kern = gemv_bf16_kernel<TT, R>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    int blocks = (N + 8 * R - 1) / (8 * R);
    const int cap = 148 * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    sl_launch(kern, dim3(blocks, tiles), 256, smem, s, y, (const bf16*)x, (const bf16*)W, T, N, K, ldx, out_f32, nullptr);
    return SL_LAUNCH_CHECK();
}

// Rows per warp: enough warps to cover the SMs a few times over, otherwise fewer rows each.
template <int TT>
static int launch_gemv_bf16(void* y, const void* x, const void* W, int T, int N, int K, int ldx, int out_f32, cudaStream_t s) {
    if (N <= 1024 && K >= 2048) {
        sl_launch(gemv_bf16_rowblock_kernel<TT>, dim3(N, (T + TT - 1) / TT), 256, 0, s, y, (const bf16*)x, (const bf16*)W, T, N, K, ldx, out_f32);
        return SL_LAUNCH_CHECK();
    }
    if (N < 148 * 8 && K >= 1024) {          // few rows: one block per row keeps every SM busy
        sl_launch(gemv_bf16_rowblock_kernel<TT>, dim3(N, (T + TT - 1) / TT), 256, 0, s, y, (const bf16*)x, (const bf16*)W, T, N, K, ldx, out_f32);
        return SL_LAUNCH_CHECK();
    }
    constexpr int RMAX = (TT >= 4) ? 2 : 4;
    if (RMAX >= 4 && N >= 148 * 8 * 4 * 2) return launch_gemv_bf16_r<TT, RMAX>(y, x, W, T, N, K, ldx, out_f32, s);
    if (N >= 148 * 8 * 2 * 2) return launch_gemv_bf16_r<TT, 2>(y, x, W, T, N, K, ldx, out_f32, s);
    return launch_gemv_bf16_r<TT, 1>(y, x, W, T, N, K, ldx, out_f32, s);
}

SL_API int sl_gemv_bf16(void* y, const void* x, const void* W, int T, int N, int K, int ldx, int out_f32, cudaStream_t s) {
    if (T == 0 || N == 0) return 0;
    if (K % 8 != 0 || ldx % 8 != 0) return -1;
    if (T == 1) return launch_gemv_bf16<1>(y, x, W, T, N, K, ldx, out_f32, s);
    if (T == 2) return launch_gemv_bf16<2>(y, x, W, T, N, K, ldx, out_f32, s);
    if (T <= 4) return launch_gemv_bf16<4>(y, x, W, T, N, K, ldx, out_f32, s);
    return launch_gemv_bf16<8>(y, x, W, T, N, K, ldx, out_f32, s);
}

// ---------------------------------------------------------------------------------------------
// NVFP4 row dot products.  A lane reads 16 bytes (32 codes) of R rows per step, the two
// UE4M3 block scales that cover them, and 32 activations per token from shared memory (fp16).
// acc[r][tt] += sum_{32} e2m1 * scale * x
template <int TT, int R>
__device__ __forceinline__ void nvfp4_rows_dot(float (&acc)[R][TT], const uint8_t* __restrict__ Wp, const uint8_t* __restrict__ S,
                                               size_t w_stride, size_t s_stride, int rows_valid, int K,
                                               const __half* __restrict__ xs, int lane) {
    // software pipeline: the loads of step i+1 are in flight while step i is expanded and multiplied
    uint4 w[R], wn[R];
    uint16_t sc[R], scn[R];
    int k = lane * 32;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        w[r] = make_uint4(0, 0, 0, 0); sc[r] = 0;
        if (k < K && r < rows_valid) {
            w[r] = ldg_nc_16(Wp + (size_t)r * w_stride + (k >> 1));
            sc[r] = *reinterpret_cast<const uint16_t*>(S + (size_t)r * s_stride + (k >> 4));
        }
    }
    for (; k < K; k += 1024) {
        const int kn = k + 1024;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            wn[r] = make_uint4(0, 0, 0, 0); scn[r] = 0;
            if (kn < K && r < rows_valid) {
                wn[r] = ldg_nc_16(Wp + (size_t)r * w_stride + (kn >> 1));
                scn[r] = *reinterpret_cast<const uint16_t*>(S + (size_t)r * s_stride + (kn >> 4));
            }
        }
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
            const uint4* xp = reinterpret_cast<const uint4*>(xs + (size_t)tt * K + k);
            __half2 xv[16];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint4 u = xp[q];
                xv[q * 4 + 0] = *reinterpret_cast<const __half2*>(&u.x);
                xv[q * 4 + 1] = *reinterpret_cast<const __half2*>(&u.y);
                xv[q * 4 + 2] = *reinterpret_cast<const __half2*>(&u.z);
                xv[q * 4 + 3] = *reinterpret_cast<const __half2*>(&u.w);
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint32_t words[4] = {w[r].x, w[r].y, w[r].z, w[r].w};
                const float2 s2 = e4m3x2_to_float2(sc[r]);
                // 16 values per scale block (words 0,1 -> scale .x ; words 2,3 -> scale .y): the 8
                // products of a block are summed as half2 pairs, then once in fp32 with the scale
                __half2 hb[2];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    __half2 wv[4];
                    e2m1x8_to_half2x4(words[q], wv);
                    __half2 a = (q & 1) ? hb[q >> 1] : __hmul2(wv[0], xv[q * 4 + 0]);
                    if (q & 1) a = __hfma2(wv[0], xv[q * 4 + 0], a);
                    a = __hfma2(wv[1], xv[q * 4 + 1], a);
                    a = __hfma2(wv[2], xv[q * 4 + 2], a);
                    a = __hfma2(wv[3], xv[q * 4 + 3], a);
                    hb[q >> 1] = a;
                }
                const float2 f0 = __half22float2(hb[0]), f1 = __half22float2(hb[1]);
                acc[r][tt] += (f0.x + f0.y) * s2.x + (f1.x + f1.y) * s2.y;
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) { w[r] = wn[r]; sc[r] = scn[r]; }
    }
}

// Stage TT activation rows as fp16 in shared memory (zero rows past T).
template <int TT>
__device__ __forceinline__ void stage_x_half(__half* xs, const bf16* x, int t0, int T, int K, int ldx) {
    for (int i = threadIdx.x; i < TT * (K / 2); i += blockDim.x) {
        const int tt = i / (K / 2), c = i % (K / 2);
        float2 f = make_float2(0.f, 0.f);
        if (t0 + tt < T) f = bf162_to_f2(*reinterpret_cast<const uint32_t*>(x + (size_t)(t0 + tt) * ldx + c * 2));
        reinterpret_cast<__half2*>(xs)[i] = __floats2half2_rn(f.x, f.y);
    }
}

// y[t, n] = g * sum_k x[t,k] * e2m1(Wp[n,k]) * e4m3(S[n, k/16])
template <int TT, int R>
__global__ void __launch_bounds__(256) gemv_nvfp4_kernel(void* __restrict__ y, const bf16* __restrict__ x,
                                                         const uint8_t* __restrict__ Wp, const uint8_t* __restrict__ S,
                                                         const float* __restrict__ gscale, int T, int N, int K, int ldx,
                                                         int out_f32) {
    PDL_ENTRY_WITH_PREFETCH({
        const int first = blockIdx.x * 8 * R;
        if (first < N) {
            prefetch_l2_rows(Wp + (size_t)first * (K / 2), min(8 * R, N - first), (size_t)K / 2);
            prefetch_l2_rows(S + (size_t)first * (K / 16), min(8 * R, N - first), (size_t)K / 16);
        }
    });
    extern __shared__ __align__(16) unsigned char smraw[];
    __half* xs = reinterpret_cast<__half*>(smraw);
    const int t0 = blockIdx.y * TT;
    stage_x_half<TT>(xs, x, t0, T, K, ldx);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
    const float g = gscale ? *gscale : 1.f;
    for (int n0 = warp * R; n0 < N; n0 += nwarps * R) {
        float acc[R][TT];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) acc[r][tt] = 0.f;
        nvfp4_rows_dot<TT, R>(acc, Wp + (size_t)n0 * (K / 2), S + (size_t)n0 * (K / 16), K / 2, K / 16,
                              min(R, N - n0), K, xs, lane);
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) {
                const float v = warp_sum(acc[r][tt]) * g;
                if (lane == 0 && n0 + r < N && t0 + tt < T) {
                    if (out_f32) ((float*)y)[(size_t)(t0 + tt) * N + n0 + r] = v;
                    else ((bf16*)y)[(size_t)(t0 + tt) * N + n0 + r] = __float2bfloat16(v);
                }
            }
    }
}

template <int TT, int R>
static int launch_gemv_nvfp4_r(void* y, const void* x, const void* Wp, const void* S, const void* g, int T, int N, int K,
                               int ldx, int out_f32, cudaStream_t s) {
    const size_t smem = (size_t)TT * K * sizeof(__half);
    auto kern = gemv_nvfp4_kernel<TT, R>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    int blocks = (N + 8 * R - 1) / (8 * R);
    if (blocks > 148 * 8) blocks = 148 * 8;
    sl_launch(kern, dim3(blocks, (T + TT - 1) / TT), 256, smem, s, y, (const bf16*)x, (const uint8_t*)Wp, (const uint8_t*)S,
                                                            (const float*)g, T, N, K, ldx, out_f32);
    return SL_LAUNCH_CHECK();
}

template <int TT>
static int launch_gemv_nvfp4(void* y, const void* x, const void* Wp, const void* S, const void* g, int T, int N, int K,
                             int ldx, int out_f32, cudaStream_t s) {
    constexpr int RMAX = (TT >= 4) ? 2 : 4;
    if (RMAX >= 4 && N >= 148 * 8 * 4 * 2) return launch_gemv_nvfp4_r<TT, RMAX>(y, x, Wp, S, g, T, N, K, ldx, out_f32, s);
    if (N >= 148 * 8 * 2 * 2) return launch_gemv_nvfp4_r<TT, 2>(y, x, Wp, S, g, T, N, K, ldx, out_f32, s);
    return launch_gemv_nvfp4_r<TT, 1>(y, x, Wp, S, g, T, N, K, ldx, out_f32, s);
}

SL_API int sl_gemv_nvfp4(void* y, const void* x, const void* Wp, const void* S, const void* g, int T, int N, int K, int ldx,
                         int out_f32, cudaStream_t s) {
    if (T == 0 || N == 0) return 0;
    if (K % 32 != 0 || ldx % 2 != 0) return -1;
    if (T == 1) return launch_gemv_nvfp4<1>(y, x, Wp, S, g, T, N, K, ldx, out_f32, s);
    if (T == 2) return launch_gemv_nvfp4<2>(y, x, Wp, S, g, T, N, K, ldx, out_f32, s);
    return launch_gemv_nvfp4<4>(y, x, Wp, S, g, T, N, K, ldx, out_f32, s);
}

// ---------------------------------------------------------------------------------------------
// MoE decode, stage 1: for each route (token t, choice j) with expert e:
//   act[route, i] = silu(g13[e,0] * W13[e, i, :] . x_t) * (g13[e,1] * W13[e, I + i, :] . x_t)
// Routes are (T * top_k) routed entries followed, when `shared` weights are given, by T shared
// entries (expert 0 of the shared stack).  grid (row tiles, routes); one block stages x_t once.
struct MoeGateUpParams {
    const bf16* x; int ldx;
    const int* ids;            // [T, top_k] global expert ids
    int T, top_k, H, I;        // I = this rank's intermediate size
    int expert_offset, num_local;   // experts held: [offset, offset + num_local)
    const uint8_t *w13, *s13; const float* g13;        // [E, 2I, H/2], [E, 2I, H/16], [E, 2]
    const uint8_t *sw13, *ss13; const float* sg13;     // shared stack (E = 1) or null
    bf16* act;                 // [T*top_k (+T), I]
};

__global__ void __launch_bounds__(256) moe_gate_up_kernel(MoeGateUpParams p) {
    pdl_grid_sync();
    extern __shared__ __align__(16) unsigned char smraw[];
    __half* xs = reinterpret_cast<__half*>(smraw);
    const int route = blockIdx.y;
    const int n_routed = p.T * p.top_k;
    int t, e;
    const uint8_t *W, *S; const float* G;
    if (route < n_routed) {
        t = route / p.top_k;
        e = p.ids[route] - p.expert_offset;
        if (e < 0 || e >= p.num_local) {       // expert lives on another rank (EP) or padding: zero row
            for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < p.I; i += gridDim.x * blockDim.x)
                p.act[(size_t)route * p.I + i] = __float2bfloat16(0.f);
            return;
        }
        W = p.w13 + (size_t)e * 2 * p.I * (p.H / 2);
        S = p.s13 + (size_t)e * 2 * p.I * (p.H / 16);
        G = p.g13 + (size_t)e * 2;
    } else {
        t = route - n_routed;
        W = p.sw13; S = p.ss13; G = p.sg13;
    }
    stage_x_half<1>(xs, p.x, t, p.T, p.H, p.ldx);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
    const float gg = G[0], gu = G[1];
    constexpr int R = 2;
    for (int i0 = warp * R; i0 < p.I; i0 += nwarps * R) {
        float ag[R][1], au[R][1];
#pragma unroll
        for (int r = 0; r < R; ++r) ag[r][0] = au[r][0] = 0.f;
        const int rv = min(R, p.I - i0);
        nvfp4_rows_dot<1, R>(ag, W + (size_t)i0 * (p.H / 2), S + (size_t)i0 * (p.H / 16), p.H / 2, p.H / 16, rv, p.H, xs, lane);
        nvfp4_rows_dot<1, R>(au, W + (size_t)(p.I + i0) * (p.H / 2), S + (size_t)(p.I + i0) * (p.H / 16), p.H / 2, p.H / 16, rv,
                             p.H, xs, lane);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float g = warp_sum(ag[r][0]) * gg, u = warp_sum(au[r][0]) * gu;
            if (lane == 0 && r < rv) p.act[(size_t)route * p.I + i0 + r] = __float2bfloat16(g / (1.f + __expf(-g)) * u);
        }
    }
}

SL_API int sl_moe_gate_up(const MoeGateUpParams* p, cudaStream_t s) {
    const int routes = p->T * p->top_k + (p->sw13 ? p->T : 0);
    if (routes == 0) return 0;
    if (p->H % 32 != 0) return -1;
    const size_t smem = (size_t)p->H * sizeof(__half);
    int bx = (p->I + 15) / 16;                // 8 warps x 2 rows per block pass
    if (bx > 64) bx = 64;
    sl_launch(moe_gate_up_kernel, dim3(bx, routes), 256, smem, s, *p);
    return SL_LAUNCH_CHECK();
}

// MoE decode, stage 2: out[t, n] = sum_j wt[t,j] * g2[e_j] * W2[e_j, n, :] . act[route(t,j), :]  (+ shared route)
// grid (row tiles, T).  All routes of token t are staged in shared memory once.
struct MoeDownParams {
    const bf16* act;           // [T*top_k (+T), I]
    const int* ids; const float* wts;
    int T, top_k, H, I, expert_offset, num_local;
    const uint8_t *w2, *s2; const float* g2;           // [E, H, I/2], [E, H, I/16], [E]
    const uint8_t *sw2, *ss2; const float* sg2;
    void* out; int out_f32;    // [T, H]
    int accumulate;            // add into out (fp32 only)
};

__global__ void __launch_bounds__(256) moe_down_kernel(MoeDownParams p, int use_push, PushCtx push) {
    pdl_grid_sync();
    // grid (H / 32, T).  The block owns 32 output rows of one token; warp w streams the rows of
    // routes w, w+8, ... (independent weight streams), the partial sums meet in shared memory.
    extern __shared__ __align__(16) unsigned char smraw[];
    __half* xs = reinterpret_cast<__half*>(smraw);                 // [routes_of_t][I]
    __shared__ float red[8][32];
    const int t = blockIdx.y;
    const int nr = p.top_k + (p.sw2 ? 1 : 0);
    for (int i = threadIdx.x; i < nr * (p.I / 2); i += blockDim.x) {
        const int j = i / (p.I / 2), c = i % (p.I / 2);
        const size_t route = (j < p.top_k) ? (size_t)t * p.top_k + j : (size_t)p.T * p.top_k + t;
        const float2 f = bf162_to_f2(*reinterpret_cast<const uint32_t*>(p.act + route * p.I + c * 2));
        reinterpret_cast<__half2*>(xs)[i] = __floats2half2_rn(f.x, f.y);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n0 = blockIdx.x * 32;
    constexpr int R = 4;
    float tot[8];                                   // rows n0 + pass*4 + r live in lane (pass*4 + r)
#pragma unroll
    for (int i = 0; i < 8; ++i) tot[i] = 0.f;
    float mine = 0.f;                               // lane l keeps the total of row n0 + l
    for (int j = warp; j < nr; j += 8) {
        const uint8_t *W, *S; float wj;
        if (j < p.top_k) {
            const int e = p.ids[(size_t)t * p.top_k + j] - p.expert_offset;
            if (e < 0 || e >= p.num_local) continue;
            W = p.w2 + (size_t)e * p.H * (p.I / 2);
            S = p.s2 + (size_t)e * p.H * (p.I / 16);
            wj = p.wts[(size_t)t * p.top_k + j] * p.g2[e];
        } else {
            W = p.sw2; S = p.ss2; wj = p.sg2[0];
        }
#pragma unroll
        for (int pass = 0; pass < 8; ++pass) {
            const int r0 = n0 + pass * R;
            if (r0 >= p.H) break;
            float acc[R][1];
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r][0] = 0.f;
            nvfp4_rows_dot<1, R>(acc, W + (size_t)r0 * (p.I / 2), S + (size_t)r0 * (p.I / 16), p.I / 2, p.I / 16,
                                 min(R, p.H - r0), p.I, xs + (size_t)j * p.I, lane);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float v = warp_sum(acc[r][0]) * wj;
                if (lane == pass * R + r) mine += v;
            }
        }
    }
    (void)tot;
    red[warp][lane] = mine;
    __syncthreads();
    if (warp == 0 && n0 + lane < p.H) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += red[w][lane];
        const size_t o = (size_t)t * p.H + n0 + lane;
        if (use_push) {
            push_store_all(push, t, n0 + lane, v, push_tag(push));
        } else if (p.out_f32) ((float*)p.out)[o] = p.accumulate ? ((float*)p.out)[o] + v : v;
        else ((bf16*)p.out)[o] = __float2bfloat16(v);
    }
}

SL_API int sl_moe_down(const MoeDownParams* p, cudaStream_t s) {
    if (p->T == 0) return 0;
    if (p->I % 32 != 0) return -1;
    const int nr = p->top_k + (p->sw2 ? 1 : 0);
    const size_t smem = (size_t)nr * p->I * sizeof(__half);
    if (smem > 200 * 1024) return -2;
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int bx = (p->H + 31) / 32;          // 32 rows per block
    sl_launch(moe_down_kernel, dim3(bx, p->T), 256, smem, s, *p, 0, PushCtx{});
    return SL_LAUNCH_CHECK();
}

// Down projection whose result rows go to every rank's receive slot (fused all-reduce producer).
SL_API int sl_moe_down_push(const MoeDownParams* p, const PushCtx* push, cudaStream_t s) {
    if (p->T == 0) return 0;
    if (p->I % 32 != 0 || push == nullptr || p->T > push->slot_rows || p->H > push->row_len) return -1;
    const int nr = p->top_k + (p->sw2 ? 1 : 0);
    const size_t smem = (size_t)nr * p->I * sizeof(__half);
    if (smem > 200 * 1024) return -2;
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int bx = (p->H + 31) / 32;
    sl_launch(moe_down_kernel, dim3(bx, p->T), 256, smem, s, *p, 1, *push);
    return SL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// NVFP4 -> bf16 expansion of stacked matrices: out[m, n, k] = e2m1 * e4m3 block scale * global scale, where the
// global scale of row n of matrix m is g[m * g_per + (n >= split ? 1 : 0)] (gate / up halves of a fused W13).
// Feeds the tcgen05 grouped GEMMs of the prefill path.  grid-stride over 32-value groups.
__global__ void nvfp4_dequant_bf16_kernel(bf16* __restrict__ out, const uint8_t* __restrict__ Wp, const uint8_t* __restrict__ S,
                                          const float* __restrict__ g, int mats, int N, int K, int g_per, int split) {
    pdl_grid_sync();
    const size_t groups = (size_t)mats * N * (K / 32);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < groups; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / (K / 32);
        const int kg = (int)(i % (K / 32));
        const int m = (int)(row / N), n = (int)(row % N);
        const float gs = g ? g[(size_t)m * g_per + ((g_per > 1 && n >= split) ? 1 : 0)] : 1.f;
        const uint4 w = ldg_nc_16(Wp + row * (K / 2) + kg * 16);
        const float2 sc = e4m3x2_to_float2(*reinterpret_cast<const uint16_t*>(S + row * (K / 16) + kg * 2));
        const uint32_t words[4] = {w.x, w.y, w.z, w.w};
        uint32_t o[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            __half2 h[4];
            e2m1x8_to_half2x4(words[q], h);
            const float s = (q < 2 ? sc.x : sc.y) * gs;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]);
                o[q * 4 + j] = f2_to_bf162(f.x * s, f.y * s);
            }
        }
        uint4* dst = reinterpret_cast<uint4*>(out + row * K + kg * 32);
#pragma unroll
        for (int q = 0; q < 4; ++q) dst[q] = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
    }
}

SL_API int sl_nvfp4_dequant_bf16(void* out, const void* Wp, const void* S, const void* g, int mats, int N, int K, int g_per,
                                 int split, cudaStream_t s) {
    if (mats == 0 || N == 0) return 0;
    if (K % 32 != 0) return -1;
    const size_t groups = (size_t)mats * N * (K / 32);
    int blocks = (int)((groups + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    sl_launch(nvfp4_dequant_bf16_kernel, blocks, 256, 0, s, (bf16*)out, (const uint8_t*)Wp, (const uint8_t*)S, (const float*)g, mats, N, K,
                                                     g_per, split);
    return SL_LAUNCH_CHECK();
}

// out[tok[r], :] += w[r] * y[r, :]   (weighted scatter of expert-sorted rows back to token order; fp32 atomics-free
// because each block owns one output token: rows of a token are found through `token_rows` [T, k] indices)
__global__ void moe_unsort_reduce_kernel(float* __restrict__ out, const void* __restrict__ y, const int* __restrict__ rows_of,
                                         const float* __restrict__ wts, int k, int H, int accumulate, int y_bf16) {
    pdl_grid_sync();
    const int t = blockIdx.y;
    for (int n = blockIdx.x * blockDim.x + threadIdx.x; n < H; n += gridDim.x * blockDim.x) {
        float v = accumulate ? out[(size_t)t * H + n] : 0.f;
        for (int j = 0; j < k; ++j) {
            const int r = rows_of[t * k + j];
            if (r >= 0)
                v += wts[t * k + j] * (y_bf16 ? __bfloat162float(((const bf16*)y)[(size_t)r * H + n]) : ((const float*)y)[(size_t)r * H + n]);
        }
        out[(size_t)t * H + n] = v;
    }
}

// Same for bf16 rows with H a multiple of 8: a thread owns 8 columns (16-byte loads, all rows of the token in flight).
__global__ void __launch_bounds__(256) moe_unsort_reduce_bf16x8_kernel(float* __restrict__ out, const bf16* __restrict__ y,
                                                                       const int* __restrict__ rows_of, const float* __restrict__ wts,
                                                                       int k, int H, int accumulate) {
    pdl_grid_sync();
    const int t = blockIdx.y;
    const int n = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (n >= H) return;
    float v[8];
    float* o = out + (size_t)t * H + n;
    if (accumulate) {
        const float4 a = *reinterpret_cast<const float4*>(o), b = *reinterpret_cast<const float4*>(o + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    for (int j0 = 0; j0 < k; j0 += 8) {
        uint4 u[8];
        float w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int r = j0 + j < k ? rows_of[t * k + j0 + j] : -1;
            w[j] = r >= 0 ? wts[t * k + j0 + j] : 0.f;
            u[j] = r >= 0 ? ldg_nc_16(y + (size_t)r * H + n) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float2 a = bf162_to_f2(u[j].x), b = bf162_to_f2(u[j].y), c = bf162_to_f2(u[j].z), d = bf162_to_f2(u[j].w);
            v[0] += w[j] * a.x; v[1] += w[j] * a.y; v[2] += w[j] * b.x; v[3] += w[j] * b.y;
            v[4] += w[j] * c.x; v[5] += w[j] * c.y; v[6] += w[j] * d.x; v[7] += w[j] * d.y;
        }
    }
    *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(o + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

SL_API int sl_moe_unsort_reduce(void* out, const void* y, const void* rows_of, const void* wts, int T, int k, int H, int accumulate,
                                int y_bf16, cudaStream_t s) {
    if (T == 0) return 0;
    if (y_bf16 && H % 8 == 0) {
        sl_launch(moe_unsort_reduce_bf16x8_kernel, dim3((H / 8 + 255) / 256, T), 256, 0, s, (float*)out, (const bf16*)y,
                  (const int*)rows_of, (const float*)wts, k, H, accumulate);
        return SL_LAUNCH_CHECK();
    }
    sl_launch(moe_unsort_reduce_kernel, dim3((H + 255) / 256, T), 256, 0, s, (float*)out, y, (const int*)rows_of,
                                                                     (const float*)wts, k, H, accumulate, y_bf16);
    return SL_LAUNCH_CHECK();
}
