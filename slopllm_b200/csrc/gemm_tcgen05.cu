// Dense GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] * B[N,K]^T, bf16 inputs,
// fp32 accumulation in TMEM, bf16 or fp32 output.
//
// Warp-specialised CTA of 192 threads per 128 x BN output tile:
//   warp 0   TMA producer: 128-byte-swizzled K-major tiles of A and B into a multi-stage ring
//   warp 1   allocates TMEM, one elected lane issues tcgen05.mma (M=128, N=BN, K=16 per
//            instruction, 4 per 64-wide K block), commits release the ring slots
//   warps 2-5 epilogue: tcgen05.ld the accumulator (one TMEM lane == one output row per thread)
//            and store
// Large GEMMs and grouped GEMMs run persistently (one CTA per SM walks the tiles) with two TMEM accumulators, so a
// tile's epilogue overlaps the next tile's loads and MMAs; the small-T weight-streaming forms launch one tile per CTA.
// No cluster multicast is used anywhere.  All mbarrier waits are bounded; on expiry the kernel
// records an error code, still frees its TMEM and returns.
//
// This replaces the reference's cuBLASLt path for batch >= 3 (`csrc/glm_gemv.cu:1642-1770`) and
// its `mma.sync` grouped kernels (`csrc/glm_mma_moe.cu:110`).
#include <algorithm>

#include "tcgen05.cuh"
#include "push.cuh"

namespace {

constexpr int BM = 128, BK = 64;

template <int BN>
struct GemmCfg {
    static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    static constexpr int STAGES = (BN >= 256) ? 4 : (BN <= 32 ? 5 : 6);   // BN=32: two CTAs per SM
    static constexpr int SMEM = STAGES * (A_BYTES + B_BYTES) + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BN>
__global__ void __launch_bounds__(192) gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA,
                                                        const __grid_constant__ CUtensorMap tmB, void* __restrict__ C,
                                                        int M, int N, int K, int ldc, int out_f32, int transpose_out,
                                                        int* __restrict__ err, int use_push, PushCtx push,
                                                        const int4* __restrict__ tiles, const int* __restrict__ num_tiles,
                                                        int kb_per_split, long long split_stride, int tiles_n, int total_tiles,
                                                        int a_group_cols, int a_group_stride) {
    using Cfg = GemmCfg<BN>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * Cfg::A_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(sB + STAGES * Cfg::B_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* tmem_full = empty + STAGES;      // [2] accumulator buffer written (MMA warp -> epilogue)
    uint64_t* tmem_empty = tmem_full + 2;      // [2] accumulator buffer read out (epilogue -> MMA warp)
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Set-up touches no global memory, so it runs while the preceding kernel is still finishing.
    if (warp == 0 && lane == 0) {
        tc::tma_prefetch_desc(&tmA);
        tc::tma_prefetch_desc(&tmB);
        for (int s = 0; s < STAGES; ++s) { tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { tc::mbar_init(&tmem_full[b], 1); tc::mbar_init(&tmem_empty[b], 4); }
        tc::mbar_fence_init();
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_holder, 2 * BN);   // two accumulators: the epilogue of a tile overlaps the next tile's MMAs
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    // Swap-AB weight streaming: operand A is the weight matrix, which no kernel of the step writes, so (SL_PDL_MODE 2)
    // the producer starts the first ring of weight tiles before waiting for the predecessor's activations.
    int pre = 0;
#if SL_PDL_MODE == 2
    pdl_trigger();
    if (transpose_out && tiles == nullptr && tiles_n == 0 && warp == 0 && lane == 0) {
        const int tkb = (K + BK - 1) / BK;
        const int k0 = kb_per_split > 0 ? (int)blockIdx.z * kb_per_split : 0;
        const int nkb = kb_per_split > 0 ? max(0, min(kb_per_split, tkb - k0)) : tkb;
        pre = min(STAGES, nkb);
        for (int kb = 0; kb < pre; ++kb) {
            tc::mbar_expect_tx(&full[kb], Cfg::A_BYTES + Cfg::B_BYTES);
            tc::tma_load_2d(sA + kb * Cfg::A_BYTES, &tmA, &full[kb], (k0 + kb) * BK, (int)blockIdx.y * BM);
        }
    }
    pdl_wait();
#else
    pdl_grid_sync();
#endif

    // Tiles of this CTA.  One-tile launch: tile (blockIdx.y, blockIdx.x).  Persistent launch (tiles_n > 0): tiles
    // blockIdx.x, blockIdx.x + gridDim.x, ... of the row-major tile grid.  Grouped GEMM: the same walk over a tile table
    // whose entries are {first A row, end of the group's A rows, first B row of the group, output column}; rows at or
    // beyond the group's end belong to the next group and are not stored.
    int first = 0, total = 1, stride = 1;
    if (tiles != nullptr) { total = *num_tiles; first = blockIdx.x; stride = gridDim.x; }
    else if (tiles_n > 0) { total = total_tiles; first = blockIdx.x; stride = gridDim.x; }
    auto tile_coords = [&](int tile, int& m0, int& n0, int& b_row0, int& m_end) {
        if (tiles != nullptr) {
            const int4 t = tiles[tile];
            m0 = t.x; m_end = t.y; b_row0 = t.z + t.w; n0 = t.w;
        } else if (tiles_n > 0) {
            m0 = (tile / tiles_n) * BM; n0 = (tile % tiles_n) * BN; b_row0 = n0; m_end = M;
        } else {
            m0 = blockIdx.y * BM; n0 = blockIdx.x * BN; b_row0 = n0; m_end = M;
        }
    };
    // split-K: blockIdx.z owns K blocks [kb0, kb0 + num_kb) and its own fp32 output slab
    const int total_kb = (K + BK - 1) / BK;
    const int kb0 = kb_per_split > 0 ? (int)blockIdx.z * kb_per_split : 0;
    const int num_kb = kb_per_split > 0 ? max(0, min(kb_per_split, total_kb - kb0)) : total_kb;
    if (kb_per_split > 0) C = (void*)((float*)C + (size_t)blockIdx.z * split_stride);

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;                      // K blocks issued so far: ring slot and phase run across tiles
            bool ok = true;
            for (int tile = first; tile < total && ok; tile += stride) {
                int m0, n0, b_row0, m_end;
                tile_coords(tile, m0, n0, b_row0, m_end);
                // batched product (one B matrix per group of output columns): the group's A columns start here
                const int a_c0 = a_group_cols > 0 ? (n0 / a_group_cols) * a_group_stride : 0;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (it < pre) {           // weight tile already in flight (issued before the dependency wait)
                        tc::tma_load_2d(sB + s * Cfg::B_BYTES, &tmB, &full[s], (kb0 + kb) * BK, b_row0);
                        continue;
                    }
                    if (!tc::mbar_wait(&empty[s], ph ^ 1)) { atomicExch(err, 1); ok = false; break; }
                    tc::mbar_expect_tx(&full[s], Cfg::A_BYTES + Cfg::B_BYTES);
                    tc::tma_load_2d(sA + s * Cfg::A_BYTES, &tmA, &full[s], a_c0 + (kb0 + kb) * BK, m0);
                    tc::tma_load_2d(sB + s * Cfg::B_BYTES, &tmB, &full[s], (kb0 + kb) * BK, b_row0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = tc::idesc_f16(BM, BN, 1);
            bool ok = true;
            int it = 0, lt = 0;
            for (int tile = first; tile < total && ok; tile += stride, ++lt) {
                const int buf = lt & 1;
                // the epilogue must have read this accumulator's previous tile (passes at once for the first two tiles)
                if (!tc::mbar_wait(&tmem_empty[buf], ((lt >> 1) & 1) ^ 1)) { atomicExch(err, 4); ok = false; break; }
                tc::fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!tc::mbar_wait(&full[s], ph)) { atomicExch(err, 2); ok = false; break; }
                    tc::fence_after_sync();
                    const uint32_t a_addr = tc::smem_u32(sA + s * Cfg::A_BYTES), b_addr = tc::smem_u32(sB + s * Cfg::B_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = tc::smem_desc_sw128(a_addr + k * 32), bd = tc::smem_desc_sw128(b_addr + k * 32);
                        tc::mma_f16_ss(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    tc::mma_commit(&empty[s]);
                }
                if (ok) tc::mma_commit(&tmem_full[buf]);   // arrives when every MMA above has finished (at once if none)
            }
            pdl_trigger_late();
        }
    } else {
        const int q = warp & 3;               // TMEM lane quarter this warp may access
        const uint32_t ptag = use_push == 1 ? push_tag(push) : 0u;
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
            const int row = m0 + q * 32 + lane;
            const uint32_t t_acc = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            auto store_chunk = [&](const uint32_t (&r)[32], int col) {
                if (transpose_out) {
                    // swap-AB use: tile rows are output features, tile columns are token rows;
                    // C is [N, M] row-major (row stride ldc), a warp writes 32 consecutive features
                    if (row < M) {
                        for (int i = 0; i < 32 && col + i < N; ++i) {
                            if (use_push) {
                                push_store_all(push, col + i, row, __uint_as_float(r[i]), ptag);
                            } else if (out_f32) ((float*)C)[(size_t)(col + i) * ldc + row] = __uint_as_float(r[i]);
                            else ((bf16*)C)[(size_t)(col + i) * ldc + row] = __float2bfloat16(__uint_as_float(r[i]));
                        }
                    }
                } else if (use_push == 2) {
                    // reduce-scatter producer: this rank's bf16 partial row goes to the rank that owns the row
                    // (rows [o * slot_rows, (o + 1) * slot_rows) belong to rank o), into slot `rank` of its staging
                    // area [world][slot_rows][row_len]; the host guarantees N % 32 == 0
                    if (row < m_end && col < N) {
                        const int owner = row / push.slot_rows;
                        bf16* dst = reinterpret_cast<bf16*>(push.bufs[owner]) +
                                    ((size_t)push.rank * push.slot_rows + (row - owner * push.slot_rows)) * push.row_len + col;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint4 v;
                            v.x = f2_to_bf162(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
                            v.y = f2_to_bf162(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
                            v.z = f2_to_bf162(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
                            v.w = f2_to_bf162(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
                            reinterpret_cast<uint4*>(dst)[i] = v;
                        }
                    }
                } else if (row < m_end && col < N) {
                    if (out_f32) {
                        float* dst = (float*)C + (size_t)row * ldc + col;
                        if (col + 32 <= N) {
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                reinterpret_cast<uint4*>(dst)[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
                        } else {
                            for (int i = 0; i < 32 && col + i < N; ++i) dst[i] = __uint_as_float(r[i]);
                        }
                    } else {
                        bf16* dst = (bf16*)C + (size_t)row * ldc + col;
                        if (col + 32 <= N) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                uint4 v;
                                v.x = f2_to_bf162(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
                                v.y = f2_to_bf162(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
                                v.z = f2_to_bf162(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
                                v.w = f2_to_bf162(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
                                reinterpret_cast<uint4*>(dst)[i] = v;
                            }
                        } else {
                            for (int i = 0; i < 32 && col + i < N; ++i) dst[i] = __float2bfloat16(__uint_as_float(r[i]));
                        }
                    }
                }
            };
            if constexpr (BN >= 64) {
                // two 32-column chunks per TMEM wait
#pragma unroll 1
                for (int c = 0; c < BN / 32; c += 2) {
                    uint32_t r0[32], r1[32];
                    tc::tmem_ld_32x32(t_acc + c * 32, r0);
                    tc::tmem_ld_32x32(t_acc + (c + 1) * 32, r1);
                    tc::tmem_ld_wait();
                    store_chunk(r0, n0 + c * 32);
                    store_chunk(r1, n0 + (c + 1) * 32);
                }
            } else {
                uint32_t r[32];
                tc::tmem_ld_32x32(t_acc, r);
                tc::tmem_ld_wait();
                store_chunk(r, n0);
            }
            // this warp's quarter of the accumulator is in registers / stored: hand the buffer back
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&tmem_empty[buf]);
            if (use_push == 2) {
                // tell the owner of this warp's 32 rows how many of their columns have landed (it expects
                // world * row_len per 32-row group): every lane orders its own stores, one lane adds
                const int row0 = m0 + q * 32;
                __threadfence_system();
                __syncwarp();
                if (lane == 0 && row0 < m_end) {
                    const int owner = row0 / push.slot_rows;
                    red_release_sys_add_u32(push.flags[owner] + (row0 - owner * push.slot_rows) / 32, (uint32_t)min(BN, N - n0));
                }
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, 2 * BN);
    }
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int BN>
int launch(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int out_f32,
           int transpose_out, int* err, cudaStream_t s, const PushCtx* push = nullptr, const int4* tiles = nullptr,
           const int* num_tiles = nullptr, int max_tiles = 0, int b_rows = 0, int splits = 1, long long split_stride = 0,
           bool persistent = false, int push_mode = 1, int a_group_cols = 0, int a_group_stride = 0, int a_cols = 0) {
    CUtensorMap tmA, tmB;
    int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)(a_cols ? a_cols : K), (uint64_t)lda * 2, BM, BK);
    if (rc) return rc;
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)(b_rows ? b_rows : N), (uint64_t)K, (uint64_t)ldb * 2, BN, BK);
    if (rc) return rc;
    auto kern = gemm_bf16_kernel<BN>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN>::SMEM);
        attr_set = true;
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    int tiles_n = 0, total_tiles = 0;
    if (tiles != nullptr) {
        grid = dim3(std::min(max_tiles, sm_count()), 1);          // persistent walk over the tile table
    } else if (persistent) {
        tiles_n = (int)grid.x;
        total_tiles = (int)(grid.x * grid.y);
        grid = dim3(std::min(total_tiles, sm_count()), 1);
    }
    int kb_per_split = 0;
    if (splits > 1) {
        const int total_kb = (K + BK - 1) / BK;
        kb_per_split = (total_kb + splits - 1) / splits;
        grid.z = (total_kb + kb_per_split - 1) / kb_per_split;
    }
    sl_launch(kern, grid, 192, GemmCfg<BN>::SMEM, s, tmA, tmB, C, M, N, K, ldc, out_f32, transpose_out, err, push ? push_mode : 0,
                                              push ? *push : PushCtx{}, tiles, num_tiles, kb_per_split, split_stride, tiles_n,
                                              total_tiles, a_group_cols, a_group_stride);
    return (int)cudaGetLastError();
}

}  // namespace

// Head-batched product for the MLA absorb / value-expansion steps of a prefill chunk:
//   C[t, g * n_per + n] = sum_k A[t, g * a_stride + k] * B[g * n_per + n, k]       g < groups, k < K
// A [M, >= (groups - 1) * a_stride + K] bf16 (row stride lda), B [groups * n_per, K] bf16 (each group's matrix stored
// output-major), C [M, groups * n_per] (row stride ldc).  The persistent tile walk of the plain GEMM, with the A tile's
// column origin taken from the output tile's group; n_per must be a multiple of the tile width.
// Replaces the reference's cuBLAS strided-batched calls (`csrc/glm_ops.cu`, absorb and v-expand).
SL_API int sl_gemm_bf16_tcgen05_batched(const void* A, const void* B, void* C, int M, int groups, int n_per, int K, int lda,
                                        int a_stride, int ldb, int ldc, int out_f32, void* err, cudaStream_t s) {
    if (M <= 0 || groups <= 0 || n_per <= 0 || K <= 0) return 0;
    if (K % BK != 0 || lda % 8 != 0 || ldb % 8 != 0 || a_stride % 8 != 0) return -1;        // a K tail would read the next group's columns
    if ((out_f32 ? ldc % 4 : ldc % 8) != 0) return -1;
    const int a_cols = (groups - 1) * a_stride + K;
    const int N = groups * n_per;
    if (n_per % 256 == 0)
        return launch<256>(A, B, C, M, N, K, lda, ldb, ldc, out_f32, 0, (int*)err, s, nullptr, nullptr, nullptr, 0, 0, 1, 0, true, 1, n_per, a_stride, a_cols);
    if (n_per % 128 == 0)
        return launch<128>(A, B, C, M, N, K, lda, ldb, ldc, out_f32, 0, (int*)err, s, nullptr, nullptr, nullptr, 0, 0, 1, 0, true, 1, n_per, a_stride, a_cols);
    if (n_per % 64 == 0)
        return launch<64>(A, B, C, M, N, K, lda, ldb, ldc, out_f32, 0, (int*)err, s, nullptr, nullptr, nullptr, 0, 0, 1, 0, true, 1, n_per, a_stride, a_cols);
    return -1;
}

// A [M, K] bf16 (row stride lda), B [N, K] bf16 (row stride ldb), C [M, N] (row stride ldc; bf16 or fp32).
// `err` is a device int the kernel sets to non-zero if one of its bounded waits expired.
SL_API int sl_gemm_bf16_tcgen05(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                                int out_f32, void* err, int bn, cudaStream_t s) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (K % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0) return -1;
    if ((out_f32 ? ldc % 4 : ldc % 8) != 0) return -1;
    // one CTA per SM walks the tile grid: the epilogue of a tile overlaps the loads and MMAs of the next
    if (bn == 64) return launch<64>(A, B, C, M, N, K, lda, ldb, ldc, out_f32, 0, (int*)err, s, nullptr, nullptr, nullptr, 0, 0, 1, 0, true);
    if (bn == 256) return launch<256>(A, B, C, M, N, K, lda, ldb, ldc, out_f32, 0, (int*)err, s, nullptr, nullptr, nullptr, 0, 0, 1, 0, true);
    return launch<128>(A, B, C, M, N, K, lda, ldb, ldc, out_f32, 0, (int*)err, s, nullptr, nullptr, nullptr, 0, 0, 1, 0, true);
}

// GEMM whose epilogue is the producer half of a reduce-scatter (prefill-sized M): tile rows are stored as bf16
// straight into the staging area of the rank that owns them (rank o owns rows [o * slot_rows, (o + 1) * slot_rows)),
// over NVLink for the peers, and each epilogue warp then adds the number of columns it delivered to the owner's
// counter of that 32-row group.  `rs->bufs[o]` = rank o's staging [world][slot_rows][row_len] (bf16), `rs->flags[o]`
// = its arrival counters [slot_rows / 32].  The consumer is sl_rs_reduce_ag (csrc/bulk_collective.cu).  Replaces
// GEMM + `p2p_reduce_scatter_write_kernel` (`csrc/glm_p2p.cu:560`) of the reference.
SL_API int sl_gemm_bf16_tcgen05_rs(const void* A, const void* B, int M, int N, int K, int lda, int ldb, void* err, int bn,
                                   const PushCtx* rs, cudaStream_t s) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (rs == nullptr || K % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0) return -1;
    if (N % 32 != 0 || N != rs->row_len || rs->slot_rows % 32 != 0 || M != rs->slot_rows * rs->world) return -1;
    if (bn == 256) return launch<256>(A, B, nullptr, M, N, K, lda, ldb, 0, 0, 0, (int*)err, s, rs, nullptr, nullptr, 0, 0, 1, 0, true, 2);
    return launch<128>(A, B, nullptr, M, N, K, lda, ldb, 0, 0, 0, (int*)err, s, rs, nullptr, nullptr, 0, 0, 1, 0, true, 2);
}

// Weight-streaming form for a few token rows (T <= 32): y[T, N] = x[T, K] * W[N, K]^T computed as
// (W tile of 128 features) x (all tokens): the weights are the 128-row MMA operand fed by a deep TMA
// ring, the tokens are the narrow N = 32 operand, the epilogue writes the transposed tile.
// `partials` (caller-owned fp32 scratch of at least 8 * T * N floats, may be null) enables split-K when the feature
// count alone gives too few CTAs to pull HBM bandwidth: each K split writes its own slab, a small kernel sums them.
__global__ void splitk_reduce_kernel(void* __restrict__ y, const float* __restrict__ part, int splits, size_t slab, int T, int N,
                                     int ldy, int out_f32) {
    pdl_grid_sync();
    const size_t total = (size_t)T * N;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < splits; ++s) v += part[(size_t)s * slab + i];
        const size_t t = i / N, n = i % N;
        if (out_f32) ((float*)y)[t * ldy + n] = v;
        else ((bf16*)y)[t * ldy + n] = __float2bfloat16(v);
    }
}

// Number of K splits the small-T linear uses for this shape (1 = no split).
SL_API int sl_smallT_splits(int T, int N, int K) {
    const int ctas = (N + BM - 1) / BM, total_kb = (K + BK - 1) / BK;
    int splits = 1;
    if (T > 0 && ctas < 120 && total_kb >= 8) {
        // two CTAs fit on each of the 148 SMs
        splits = (200 + ctas - 1) / ctas;
        if (splits > 8) splits = 8;
        if (splits > total_kb / 4) splits = total_kb / 4;
        // every split must own at least one K block
        const int per = (total_kb + splits - 1) / splits;
        splits = (total_kb + per - 1) / per;
    }
    return splits < 1 ? 1 : splits;
}

// `splits` must be 1 or the value of sl_smallT_splits for this shape.  With splits > 1 every K split writes an fp32
// slab [T, N] into `partials` ([splits, T, N]); if `y` is not null a small kernel then sums the slabs into it,
// otherwise the slabs are the result (the consumer adds them up).
SL_API int sl_linear_smallT_bf16_tcgen05(const void* x, const void* W, void* y, int T, int N, int K, int ldx, int ldw, int ldy,
                                         int out_f32, void* err, void* partials, int splits, cudaStream_t s) {
    if (T <= 0 || N <= 0 || K <= 0) return 0;
    if (T > 32 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return -1;
    if (splits <= 1) return launch<32>(W, x, y, N, T, K, ldw, ldx, ldy, out_f32, 1, (int*)err, s);
    if (partials == nullptr || splits != sl_smallT_splits(T, N, K)) return -1;
    const long long slab = (long long)T * N;
    int rc = launch<32>(W, x, partials, N, T, K, ldw, ldx, N, 1, 1, (int*)err, s, nullptr, nullptr, nullptr, 0, 0, splits, slab);
    if (rc || y == nullptr) return rc;
    int blocks = (int)(((size_t)T * N + 255) / 256);
    if (blocks > 148 * 4) blocks = 148 * 4;
    sl_launch(splitk_reduce_kernel, blocks, 256, 0, s, y, (const float*)partials, splits, (size_t)slab, T, N, ldy, out_f32);
    return (int)cudaGetLastError();
}

// Weight-streaming linear whose fp32 result rows go to every rank's receive slot (fused all-reduce producer).
SL_API int sl_linear_smallT_bf16_tcgen05_push(const void* x, const void* W, int T, int N, int K, int ldx, int ldw, void* err,
                                              const PushCtx* push, cudaStream_t s) {
    if (T <= 0 || N <= 0 || K <= 0) return 0;
    if (push == nullptr || T > 32 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || T > push->slot_rows || N > push->row_len) return -1;
    return launch<32>(W, x, nullptr, N, T, K, ldw, ldx, 0, 1, 1, (int*)err, s, push);
}

// Grouped GEMM over row groups of A (tokens sorted by expert): group g owns A rows [off[g], off[g+1]) and B rows
// [g*N, (g+1)*N) of the stacked weight matrix B [groups*N, K].  `tiles` is a device table of at most `max_tiles`
// entries {m0, group row end, g*N, n0} built by sl_build_group_tiles, `num_tiles` its length on the device.
// C [M, N] row-major.  Replaces the reference's sort + `grouped_mma_kernel` (`csrc/glm_mma_moe.cu:110-460`).
SL_API int sl_grouped_gemm_bf16_tcgen05(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                                        int out_f32, int groups, const void* tiles, const void* num_tiles, int max_tiles,
                                        void* err, int bn, cudaStream_t s) {
    if (M <= 0 || N <= 0 || K <= 0 || max_tiles <= 0) return 0;
    if (K % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0 || (out_f32 ? ldc % 4 : ldc % 8) != 0) return -1;
    // `bn` (128 or 256) is the column width the tile table was built with; wide tiles halve the number of CTAs
    // when the reduction is short and the per-tile set-up dominates
    if (bn == 256)
        return launch<256>(A, B, C, M, N, K, lda, ldb, ldc, out_f32, 0, (int*)err, s, nullptr, (const int4*)tiles,
                           (const int*)num_tiles, max_tiles, groups * N);
    if (bn != 128) return -1;
    return launch<128>(A, B, C, M, N, K, lda, ldb, ldc, out_f32, 0, (int*)err, s, nullptr, (const int4*)tiles,
                       (const int*)num_tiles, max_tiles, groups * N);
}

// offsets [groups + 1] (device, int32) -> tile table.  One thread per group enumerates its (row tile, column tile) pairs
// at a position given by a prefix sum over the groups' tile counts.
__global__ void build_group_tiles_kernel(int4* __restrict__ tiles, int* __restrict__ num_tiles, const int* __restrict__ offsets,
                                         int groups, int N, int max_tiles, int bn) {
    pdl_grid_sync();
    __shared__ int base[1025];
    const int g = threadIdx.x;
    const int ncol = (N + bn - 1) / bn;
    int mine = 0;
    if (g < groups) mine = ((offsets[g + 1] - offsets[g] + 127) / 128) * ncol;
    base[g + 1] = mine;
    if (g == 0) base[0] = 0;
    __syncthreads();
    if (g == 0) for (int i = 1; i <= groups; ++i) base[i] += base[i - 1];
    __syncthreads();
    if (g < groups) {
        int at = base[g];
        const int r0 = offsets[g], r1 = offsets[g + 1];
        for (int m = r0; m < r1; m += 128)
            for (int c = 0; c < ncol; ++c, ++at)
                if (at < max_tiles) tiles[at] = make_int4(m, r1, g * N, c * bn);
    }
    if (g == 0) *num_tiles = min(base[groups], max_tiles);
}

SL_API int sl_build_group_tiles(void* tiles, void* num_tiles, const void* offsets, int groups, int N, int max_tiles, int bn,
                                cudaStream_t s) {
    if (groups <= 0 || groups > 1024 || (bn != 128 && bn != 256)) return -1;
    sl_launch(build_group_tiles_kernel, 1, 1024, 0, s, (int4*)tiles, (int*)num_tiles, (const int*)offsets, groups, N, max_tiles, bn);
    return (int)cudaGetLastError();
}
