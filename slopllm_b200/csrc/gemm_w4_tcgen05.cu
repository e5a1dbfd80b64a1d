// GEMM with NVFP4 weights expanded inside the kernel (W4A16): C[M,N] = A[M,K] * W[N,K]^T * g, A in f16, W as packed
// E2M1 codes with one E4M3 scale per 16 values and an fp32 global scale g per weight matrix (two for a gate|up stack).
//
// tcgen05 has no instruction that multiplies 16-bit activations by block-scaled 4-bit weights, so the weight tile is
// turned into f16 on its way into shared memory: code x block scale is exact in f16 (1 + 3 mantissa bits, exponents
// 2^-10 .. 2^11), the global scale is applied to the output columns in the epilogue.  Persistent CTA of 704 threads per SM:
//   warp 0      TMA producer of the activation tiles (128-byte swizzle)
//   warp 1      TMEM allocation, tcgen05.mma issue (kind::f16, M = 128, N = BN, K = 16), two accumulators
//   warps 2-5   epilogue (TMEM -> registers -> global), overlaps the next tile's main loop
//   warps 6-21  weight converters: 16 packed bytes + 2 scale bytes per thread and K block from global memory (the next four
//               blocks in flight in registers), cvt.rn.f16x2.e2m1x2 + one multiply per pair, stores in the swizzled K-major
//               layout the MMA descriptor expects, generic->async proxy fence, arrive on the stage's barrier
// A stage is full when the TMA bytes have landed and all sixteen converter warps have arrived.  Every wait is bounded.
//
// Replaces, for T > 32 rows, the expansion kernel + bf16 GEMM pair (the reference's prefill path also goes through
// bf16: `csrc/glm_mma_moe_coop.cu:351` dequantises FP4 with an identity MMA before its `mma.sync` GEMM).
#include <algorithm>

#include "tcgen05.cuh"

namespace {

constexpr int BM = 128, BK = 64, CONV_WARPS = 16, THREADS = 192 + CONV_WARPS * 32;

template <int BN>
struct W4Cfg {
    static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    static constexpr int STAGES = (BN >= 256) ? 4 : 6;
    static constexpr int SMEM = STAGES * (A_BYTES + B_BYTES) + 1024 /*align*/ + 256 /*barriers*/;
};

struct W4Weights {
    const uint8_t* wq;     // [rows, K / 2]
    const uint8_t* ws;     // [rows, K / 16] e4m3
    const float* gs;       // [groups * g_per]
    int g_per, split;      // g_per == 2: output columns below `split` use gs[2 g], the others gs[2 g + 1]
    int group_rows;        // weight rows per group (N)
};

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int BN>
__global__ void __launch_bounds__(THREADS) gemm_w4_kernel(const __grid_constant__ CUtensorMap tmA, W4Weights w, void* __restrict__ C,
                                                          int M, int N, int K, int ldc, int out_kind, int* __restrict__ err,
                                                          const int4* __restrict__ tiles, const int* __restrict__ num_tiles,
                                                          int tiles_n, int total_tiles) {
    using Cfg = W4Cfg<BN>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * Cfg::A_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(sB + STAGES * Cfg::B_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* tmem_full = empty + STAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0 && lane == 0) {
        tc::tma_prefetch_desc(&tmA);
        for (int s = 0; s < STAGES; ++s) { tc::mbar_init(&full[s], 1 + CONV_WARPS); tc::mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { tc::mbar_init(&tmem_full[b], 1); tc::mbar_init(&tmem_empty[b], 4); }
        tc::mbar_fence_init();
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_holder, 2 * BN);
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    pdl_grid_sync();

    // tiles of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ... of the row-major tile grid or of the group tile table
    // ({first A row, end of the group's A rows, first weight row of the group, output column})
    const int first = blockIdx.x, stride = gridDim.x;
    const int total = tiles != nullptr ? *num_tiles : total_tiles;
    auto tile_coords = [&](int tile, int& m0, int& n0, int& b_row0, int& m_end) {
        if (tiles != nullptr) {
            const int4 t = tiles[tile];
            m0 = t.x; m_end = t.y; b_row0 = t.z; n0 = t.w;
        } else {
            m0 = (tile / tiles_n) * BM; n0 = (tile % tiles_n) * BN; b_row0 = 0; m_end = M;
        }
    };
    const int num_kb = K / BK;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int tile = first; tile < total && ok; tile += stride) {
                int m0, n0, b_row0, m_end;
                tile_coords(tile, m0, n0, b_row0, m_end);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!tc::mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1)) { atomicExch(err, 1); ok = false; break; }
                    tc::mbar_expect_tx(&full[s], Cfg::A_BYTES);
                    tc::tma_load_2d(sA + s * Cfg::A_BYTES, &tmA, &full[s], kb * BK, m0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = tc::idesc_f16(BM, BN, 0);     // f16 x f16 -> fp32
            bool ok = true;
            int it = 0, lt = 0;
            for (int tile = first; tile < total && ok; tile += stride, ++lt) {
                const int buf = lt & 1;
                if (!tc::mbar_wait(&tmem_empty[buf], ((lt >> 1) & 1) ^ 1)) { atomicExch(err, 4); ok = false; break; }
                tc::fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!tc::mbar_wait(&full[s], (it / STAGES) & 1)) { atomicExch(err, 2); ok = false; break; }
                    tc::fence_after_sync();
                    const uint32_t a_addr = tc::smem_u32(sA + s * Cfg::A_BYTES), b_addr = tc::smem_u32(sB + s * Cfg::B_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = tc::smem_desc_sw128(a_addr + k * 32), bd = tc::smem_desc_sw128(b_addr + k * 32);
                        tc::mma_f16_ss(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    tc::mma_commit(&empty[s]);
                }
                if (ok) tc::mma_commit(&tmem_full[buf]);
            }
            pdl_trigger_late();
        }
    } else if (warp < 6) {
        const int q = warp & 3;
        int lt = 0;
        for (int tile = first; tile < total; tile += stride, ++lt) {
            const int buf = lt & 1;
            if (!tc::mbar_wait(&tmem_full[buf], (lt >> 1) & 1)) {
                if (lane == 0) atomicExch(err, 3);
                break;
            }
            tc::fence_after_sync();
            int m0, n0, b_row0, m_end;
            tile_coords(tile, m0, n0, b_row0, m_end);
            const int grp = w.group_rows > 0 ? b_row0 / w.group_rows : 0;
            const int row = m0 + q * 32 + lane;
            const uint32_t t_acc = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            auto store_chunk = [&](const uint32_t (&r)[32], int col) {
                if (row >= m_end || col >= N) return;
                const float g = w.g_per == 2 ? w.gs[2 * grp + (col >= w.split ? 1 : 0)] : w.gs[grp];
                if (out_kind == 1) {
                    float* dst = (float*)C + (size_t)row * ldc + col;
                    if (col + 32 <= N) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            reinterpret_cast<float4*>(dst)[i] = make_float4(__uint_as_float(r[4 * i]) * g, __uint_as_float(r[4 * i + 1]) * g,
                                                                            __uint_as_float(r[4 * i + 2]) * g, __uint_as_float(r[4 * i + 3]) * g);
                    } else {
                        for (int i = 0; i < 32 && col + i < N; ++i) dst[i] = __uint_as_float(r[i]) * g;
                    }
                } else {
                    uint16_t* dst = (uint16_t*)C + (size_t)row * ldc + col;
                    if (col + 32 <= N) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint32_t v[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float a = __uint_as_float(r[8 * i + 2 * j]) * g, b = __uint_as_float(r[8 * i + 2 * j + 1]) * g;
                                v[j] = out_kind == 2 ? pack_h2(a, b) : f2_to_bf162(a, b);
                            }
                            reinterpret_cast<uint4*>(dst)[i] = make_uint4(v[0], v[1], v[2], v[3]);
                        }
                    } else {
                        for (int i = 0; i < 32 && col + i < N; ++i) {
                            const float a = __uint_as_float(r[i]) * g;
                            if (out_kind == 2) { __half h = __float2half_rn(a); dst[i] = *reinterpret_cast<uint16_t*>(&h); }
                            else { bf16 h = __float2bfloat16(a); dst[i] = *reinterpret_cast<uint16_t*>(&h); }
                        }
                    }
                }
            };
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r0[32];
                tc::tmem_ld_32x32(t_acc + c * 32, r0);
                tc::tmem_ld_wait();
                store_chunk(r0, n0 + c * 32);
            }
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&tmem_empty[buf]);
        }
    } else {
        // ---- weight converters ----
        // Two threads share a weight row of the tile (four for BN = 128).  A thread loads SB K blocks at a time and keeps the
        // next SB blocks in flight in registers while it converts the current ones (enough bytes on the wire per SM to cover
        // the memory latency).  Sixteen warps: the conversion is a chain of dependent integer / f16 operations, so it takes
        // about four warps per scheduler to keep the issue slots busy.
        constexpr int TPR = CONV_WARPS * 32 / BN;     // threads per weight row of the tile (2 or 4)
        constexpr int NW = 8 / TPR;                   // 32-bit words (8 codes = one 16-byte f16 chunk each) per thread and K block
        constexpr int SB = 4;                         // K blocks per load round
        static_assert(NW == 4 || NW == 2, "a thread converts 16 or 8 packed bytes per K block");
        const int ct = threadIdx.x - 192;
        const int row = ct / TPR, part = ct % TPR;   // part: which 16 / 8 bytes of the row's 32 packed bytes per K block
        const size_t q_stride = (size_t)K / 2, s_stride = (size_t)K / 16;
        uint32_t cur[SB][NW], nxt[SB][NW], cur_s[SB], nxt_s[SB];
        auto load_sb = [&](uint32_t (&dst)[SB][NW], uint32_t (&sc)[SB], int b_row0, int n0, int kb0) {
            const bool valid = n0 + row < N;
            const uint8_t* qp = w.wq + (size_t)(b_row0 + n0 + row) * q_stride + part * (NW * 4);
            const uint8_t* sp = w.ws + (size_t)(b_row0 + n0 + row) * s_stride + part * (NW / 2);
#pragma unroll
            for (int j = 0; j < SB; ++j) {
                if (valid && kb0 + j < num_kb) {
                    if constexpr (NW == 4) {
                        const uint4 v = ldg_nc_16(qp + (kb0 + j) * 32);
                        dst[j][0] = v.x; dst[j][1] = v.y; dst[j][2] = v.z; dst[j][3] = v.w;
                        sc[j] = (uint32_t)*reinterpret_cast<const uint16_t*>(sp + (kb0 + j) * 4);
                    } else {
                        const uint2 v = ldg_nc_8(qp + (kb0 + j) * 32);
                        dst[j][0] = v.x; dst[j][1] = v.y;
                        sc[j] = (uint32_t)sp[(kb0 + j) * 4];
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < NW; ++i) dst[j][i] = 0u;
                    sc[j] = 0u;
                }
            }
        };
        int tile = first, kb0 = 0, m0 = 0, n0 = 0, b_row0 = 0, m_end = 0;
        bool have = tile < total && num_kb > 0;
        if (have) {
            tile_coords(tile, m0, n0, b_row0, m_end);
            load_sb(cur, cur_s, b_row0, n0, 0);
        }
        int it = 0;
        bool ok = true;
        while (have && ok) {
            int ntile = tile, nkb0 = kb0 + SB, nn0 = n0, nb_row0 = b_row0;
            bool nhave = true;
            if (nkb0 >= num_kb) {
                nkb0 = 0;
                ntile = tile + stride;
                nhave = ntile < total;
                if (nhave) tile_coords(ntile, m0, nn0, nb_row0, m_end);
            }
            if (nhave) load_sb(nxt, nxt_s, nb_row0, nn0, nkb0);
#pragma unroll
            for (int j = 0; j < SB; ++j) {
                if (ok && kb0 + j < num_kb) {
                    const int s = it % STAGES;
                    if (!tc::mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1)) {
                        if (lane == 0) atomicExch(err, 5);
                        ok = false;
                    } else {
                        uint8_t* brow = sB + s * Cfg::B_BYTES + row * 128;
#pragma unroll
                        for (int i = 0; i < NW; ++i) {
                            __half2 h[4];
                            e2m1x8_to_half2x4(cur[j][i], h);
                            // scale of the 16-value block this word belongs to (two words per block)
                            const uint32_t sb = (cur_s[j] >> (8 * (i >> 1))) & 0xffu;
                            __half2_raw sr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(sb | (sb << 8)), __NV_E4M3);
                            const __half2 sc = *reinterpret_cast<__half2*>(&sr);
                            uint4 v;
                            __half2 p0 = __hmul2(h[0], sc), p1 = __hmul2(h[1], sc), p2 = __hmul2(h[2], sc), p3 = __hmul2(h[3], sc);
                            v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
                            v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
                            const int chunk = part * NW + i;
                            *reinterpret_cast<uint4*>(brow + ((chunk ^ (row & 7)) << 4)) = v;
                        }
                        tc::fence_proxy_async_smem();     // the MMA reads these generic-proxy stores through the async proxy
                        __syncwarp();
                        if (lane == 0) tc::mbar_arrive(&full[s]);
                        ++it;
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < SB; ++j) {
#pragma unroll
                for (int i = 0; i < NW; ++i) cur[j][i] = nxt[j][i];
                cur_s[j] = nxt_s[j];
            }
            tile = ntile; kb0 = nkb0; n0 = nn0; b_row0 = nb_row0; have = nhave;
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, 2 * BN);
    }
}

int w4_sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int BN>
int launch_w4(const void* A, const W4Weights& w, void* C, int M, int N, int K, int lda, int ldc, int out_kind, int* err,
              const int4* tiles, const int* num_tiles, int max_tiles, cudaStream_t s) {
    CUtensorMap tmA;
    const int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, BM, BK);
    if (rc) return rc;
    auto kern = gemm_w4_kernel<BN>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, W4Cfg<BN>::SMEM);
        attr_set = true;
    }
    int tiles_n = 0, total_tiles = 0, grid = 0;
    if (tiles != nullptr) {
        grid = std::min(max_tiles, w4_sm_count());
    } else {
        tiles_n = (N + BN - 1) / BN;
        total_tiles = tiles_n * ((M + BM - 1) / BM);
        grid = std::min(total_tiles, w4_sm_count());
    }
    sl_launch(kern, grid, THREADS, W4Cfg<BN>::SMEM, s, tmA, w, C, M, N, K, ldc, out_kind, err, tiles, num_tiles, tiles_n, total_tiles);
    return (int)cudaGetLastError();
}

bool w4_shape_ok(int M, int N, int K, int lda, int ldc, int out_kind) {
    if (M <= 0 || N <= 0 || K <= 0) return false;
    if (K % 64 != 0 || lda % 8 != 0) return false;                   // whole K blocks, 16-byte rows for TMA and the packed loads
    return (out_kind == 1 ? ldc % 4 : ldc % 8) == 0;
}

}  // namespace

// A [M, K] f16 (row stride lda), weights NVFP4 [N, K/2] + e4m3 [N, K/16] + fp32 global scales gs[g_per] (g_per 1 or 2; with 2,
// output columns below `split` use gs[0], the others gs[1]).  C [M, N] row stride ldc; out_kind 0 bf16, 1 fp32, 2 f16.
SL_API int sl_gemm_w4_tcgen05(const void* A, const void* wq, const void* ws, const void* gs, int g_per, int split, void* C, int M,
                              int N, int K, int lda, int ldc, int out_kind, void* err, int bn, cudaStream_t s) {
    if (M <= 0 || N <= 0) return 0;
    if (!w4_shape_ok(M, N, K, lda, ldc, out_kind) || (g_per != 1 && g_per != 2)) return -1;
    const W4Weights w{(const uint8_t*)wq, (const uint8_t*)ws, (const float*)gs, g_per, split, 0};
    if (bn == 128) return launch_w4<128>(A, w, C, M, N, K, lda, ldc, out_kind, (int*)err, nullptr, nullptr, 0, s);
    if (bn != 256) return -1;
    return launch_w4<256>(A, w, C, M, N, K, lda, ldc, out_kind, (int*)err, nullptr, nullptr, 0, s);
}

// Grouped form over expert-sorted rows of A: group g owns A rows [off[g], off[g+1]) and weight rows [g N, (g + 1) N) of the
// stacked tensors; `tiles` / `num_tiles` come from sl_build_group_tiles with the same `bn`; gs holds g_per scales per group.
SL_API int sl_grouped_gemm_w4_tcgen05(const void* A, const void* wq, const void* ws, const void* gs, int g_per, int split, void* C,
                                      int M, int N, int K, int lda, int ldc, int out_kind, const void* tiles, const void* num_tiles,
                                      int max_tiles, void* err, int bn, cudaStream_t s) {
    if (M <= 0 || N <= 0 || max_tiles <= 0) return 0;
    if (!w4_shape_ok(M, N, K, lda, ldc, out_kind) || (g_per != 1 && g_per != 2)) return -1;
    const W4Weights w{(const uint8_t*)wq, (const uint8_t*)ws, (const float*)gs, g_per, split, N};
    if (bn == 128)
        return launch_w4<128>(A, w, C, M, N, K, lda, ldc, out_kind, (int*)err, (const int4*)tiles, (const int*)num_tiles, max_tiles, s);
    if (bn != 256) return -1;
    return launch_w4<256>(A, w, C, M, N, K, lda, ldc, out_kind, (int*)err, (const int4*)tiles, (const int*)num_tiles, max_tiles, s);
}
