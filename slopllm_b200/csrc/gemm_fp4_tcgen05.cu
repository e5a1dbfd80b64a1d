// Block-scaled NVFP4 GEMM on the 5th-generation tensor cores (W4A4): both operands stay packed E2M1 from HBM to the
// tensor core, their UE4M3 scales (one per 16 elements) ride in TMEM, `tcgen05.mma.kind::mxf4nvf4.block_scale`
// multiplies and scales in one instruction, accumulators are fp32 in TMEM.  Nothing is expanded on the CUDA cores.
//
//     out[token, n] = gB[token] * gA * sum_k  W[n, k] * X[token, k]
//
// The weight matrix is the 128-row MMA operand ("A"), the activation rows are the narrow one ("B"), so the same kernel
// serves a prefill chunk (many tokens per expert) and a decode step (a handful): work is a table of tiles
// {128 weight rows (optionally paired with the matching 128 "up" rows)} x {up to BN token rows}, walked persistently by
// one CTA per SM.  Grouped use (MoE): the table names, per tile, the weight rows of one expert and the token rows that
// were routed to it.
//
// Operand formats
//   W    packed codes [rows, K/2] (two per byte, even index in the low nibble), TMA-tiled with the 128-byte swizzle
//   SFA  weight scales re-laid once at load time into 512-byte tiles of 128 rows x 4 scales, the layout `tcgen05.cp`
//        broadcasts into TMEM: byte (r % 32) * 16 + (r / 32) * 4 + (kb % 4) of tile (r / 128, kb / 4) (sl_nvfp4_sf_tiles)
//   X    packed codes [tokens, K/2] and per-row global scales gB[tokens] written by sl_nvfp4_quantize_rows
//   SFB  activation scales in the same 512-byte tiles, one per GEMM tile of BN token rows and 64 reduction indices.  A
//        group's token rows start anywhere, so the tiles are indexed by the *padded* row p = pad[g] + (m - offsets[g]),
//        where pad[] rounds every group up to a multiple of BN rows: tile p / BN, row p % BN.  Scale columns in TMEM
//        then always start at a multiple of four, which the instruction requires.
//
// Warp roles: warp 0 issues TMA / bulk copies into a multi-stage ring, warp 1 copies scales into TMEM and issues the MMAs,
// the other 4 x BN / 32 warps read the accumulators out of TMEM (one lane = one weight row; one warp per TMEM lane quarter
// and 32-column chunk: with four epilogue warps in all, one per scheduler issued at 0.3 instructions per cycle and bound
// tiles with a short reduction) and store the transposed tile.  Two accumulator buffers when TMEM allows, so a tile's epilogue overlaps the next tile's MMAs.  No cluster
// multicast.  Every wait is bounded (error code, TMEM freed, normal return).
//
// Reference counterpart: `coop_moe_kernel` (`csrc/glm_mma_moe_coop.cu:351`), which uses the warp-level block-scaled FP4
// MMA of sm_120 only to expand weights to bf16 before a bf16 MMA.
#include <algorithm>

#include "tcgen05.cuh"

namespace {

constexpr int BM = 128;            // weight rows per tile
constexpr int BKB = 128;           // bytes of packed codes per row and stage = 256 reduction indices = 4 instructions
constexpr int KSTEPS = 4;

struct Fp4Tile {
    int a_row0;                    // first weight row of the tile (the paired "up" tile starts pair_rows further)
    int sfa_blk0;                  // 128-row scale block of that row
    int b_row0, b_valid;           // first token row, number of valid token rows (<= BN)
    int out_n0, group;             // output column of weight row 0 of the tile, group (expert) for the global scales
    int sfb_tile;                  // scale tile of the token rows (padded row / BN)
    int tab0;                      // column-row table mode: entry of this tile's first token column (see Fp4Params::col_rows)
};

template <int BN, int PAIR>
struct Fp4Cfg {
    static constexpr int NA = PAIR ? 2 : 1;
    static constexpr int EPI_PER_Q = BN / 32;                 // epilogue warps per TMEM lane quarter: one per 32-column chunk
    static constexpr int EPI_WARPS = 4 * EPI_PER_Q, THREADS = (2 + EPI_WARPS) * 32;
    static constexpr int A_BYTES = BM * BKB, SF_BYTES = KSTEPS * 512, B_BYTES = BN * BKB;
    static constexpr int TX = NA * (A_BYTES + SF_BYTES) + B_BYTES + SF_BYTES;        // bytes that land per stage
    static constexpr int STAGE = (TX + 1023) / 1024 * 1024;
    static constexpr int STAGES = (200 * 1024) / STAGE > 8 ? 8 : (200 * 1024) / STAGE;
    static constexpr int SMEM = STAGES * STAGE + 1024 + 256;
    static constexpr int ACC_COLS = NA * BN;
    static constexpr int SF_COLS = (NA + 1) * 16;
    static constexpr int NBUF = (2 * ACC_COLS + SF_COLS <= 512) ? 2 : 1;
    static constexpr int TMEM_COLS = (NBUF * ACC_COLS + SF_COLS <= 64) ? 64 : (NBUF * ACC_COLS + SF_COLS <= 128) ? 128
                                     : (NBUF * ACC_COLS + SF_COLS <= 256) ? 256 : 512;
};

struct Fp4Params {
    const uint8_t* sfa;            // weight scale tiles [blocks][K/64][512]
    const uint8_t* sfb;            // activation scale tiles [tiles][K/64][512]
    const float* gA;               // [groups] or [groups][2] (PAIR: gate, up) global scales of the weights
    const float* gB;               // [tokens] global scales of the activation rows
    void* out;                     // [tokens, ldo]: bf16 / f32 (out_kind 0 / 1)
    int K, ldo, out_kind;
    int pair_rows, pair_blks;      // PAIR: distance from a gate row to its up row, in rows and in 128-row scale blocks
    const Fp4Tile* tiles; const int* num_tiles;
    int* err;
    // expert-parallel combine: when set, output row m (bf16) is not stored at out[m] but at scatter_base[meta.x] +
    // meta.y * ldo, meta = row_meta[m] = {home rank of the row's token, its route slot there} (peer memory, plain stores)
    const int2* row_meta;
    bf16* scatter_base[8];
    // column-row table (decode MoE): token column c of a tile is stored at output row col_rows[tile.tab0 + c], a negative
    // entry drops the column.  The token operand can then be the same few rows for every tile (all tokens of the step)
    // while each expert's tile keeps only the tokens routed to it, or a compact per-expert block whose rows scatter back
    // to their routes.  bf16 or f32 rows (out_kind).
    const int* col_rows;
    // second weight set, used by tiles whose group is negative (the shared expert, stored apart from the expert stack)
    const uint8_t* sfa2;
    const float* gA2;
};

template <int BN, int PAIR>
__global__ void __launch_bounds__(Fp4Cfg<BN, PAIR>::THREADS) gemm_fp4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                                       const __grid_constant__ CUtensorMap tmA2, const Fp4Params p) {
    using Cfg = Fp4Cfg<BN, PAIR>;
    constexpr int STAGES = Cfg::STAGES, NA = Cfg::NA, NBUF = Cfg::NBUF;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // stage layout: A tiles (1024-aligned) | B tile | SFA tiles | SFB tile
    auto sA = [&](int s, int a) { return smem + (size_t)s * Cfg::STAGE + (size_t)a * Cfg::A_BYTES; };
    auto sB = [&](int s) { return smem + (size_t)s * Cfg::STAGE + (size_t)NA * Cfg::A_BYTES; };
    auto sSFA = [&](int s, int a) { return smem + (size_t)s * Cfg::STAGE + (size_t)NA * Cfg::A_BYTES + Cfg::B_BYTES + (size_t)a * Cfg::SF_BYTES; };
    auto sSFB = [&](int s) { return smem + (size_t)s * Cfg::STAGE + (size_t)NA * (Cfg::A_BYTES + Cfg::SF_BYTES) + Cfg::B_BYTES; };
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)STAGES * Cfg::STAGE);
    uint64_t* empty = full + STAGES;
    uint64_t* tmem_full = empty + STAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    static_assert(Cfg::STAGE % 1024 == 0, "stages must keep the 1024-byte alignment of the swizzled tiles");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0 && lane == 0) {
        tc::tma_prefetch_desc(&tmA);
        tc::tma_prefetch_desc(&tmB);
        tc::tma_prefetch_desc(&tmA2);
        for (int s = 0; s < STAGES; ++s) { tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { tc::mbar_init(&tmem_full[b], 1); tc::mbar_init(&tmem_empty[b], Cfg::EPI_WARPS); }
        tc::mbar_fence_init();
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_holder, Cfg::TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    const uint32_t tmem_sf = tmem_base + NBUF * Cfg::ACC_COLS;          // SFA: NA x 16 columns, then SFB: 16
    pdl_grid_sync();

    const int total = *p.num_tiles;
    const int num_kb = p.K / (2 * BKB);
    const int KT = p.K / 64;                                            // scale tiles of 4 scales along K

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            Fp4Tile t_next{};
            if ((int)blockIdx.x < total) t_next = p.tiles[blockIdx.x];
            for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
                const Fp4Tile t = t_next;
                if (tile + (int)gridDim.x < total) t_next = p.tiles[tile + gridDim.x];      // in flight while this tile's loads are issued
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!tc::mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1)) { atomicExch(p.err, 11); ok = false; break; }
                    tc::mbar_expect_tx(&full[s], Cfg::TX);
                    const CUtensorMap* ta = t.group < 0 ? &tmA2 : &tmA;
                    const uint8_t* sfa = t.group < 0 ? p.sfa2 : p.sfa;
                    tc::tma_load_2d(sA(s, 0), ta, &full[s], kb * BKB, t.a_row0);
                    tc::bulk_load_1d(sSFA(s, 0), sfa + ((size_t)t.sfa_blk0 * KT + (size_t)kb * KSTEPS) * 512, Cfg::SF_BYTES, &full[s]);
                    if (PAIR) {
                        tc::tma_load_2d(sA(s, 1), ta, &full[s], kb * BKB, t.a_row0 + p.pair_rows);
                        tc::bulk_load_1d(sSFA(s, 1), sfa + ((size_t)(t.sfa_blk0 + p.pair_blks) * KT + (size_t)kb * KSTEPS) * 512, Cfg::SF_BYTES,
                                         &full[s]);
                    }
                    tc::tma_load_2d(sB(s), &tmB, &full[s], kb * BKB, t.b_row0);
                    tc::bulk_load_1d(sSFB(s), p.sfb + ((size_t)t.sfb_tile * KT + (size_t)kb * KSTEPS) * 512, Cfg::SF_BYTES, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = tc::idesc_nvf4(BM, BN);
            bool ok = true;
            int it = 0, lt = 0;
            for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++lt) {
                const int buf = NBUF == 2 ? (lt & 1) : 0;
                const uint32_t par = NBUF == 2 ? (((lt >> 1) & 1) ^ 1) : ((lt & 1) ^ 1);
                if (!tc::mbar_wait(&tmem_empty[buf], par)) { atomicExch(p.err, 14); ok = false; break; }
                tc::fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * Cfg::ACC_COLS;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!tc::mbar_wait(&full[s], (it / STAGES) & 1)) { atomicExch(p.err, 12); ok = false; break; }
                    tc::fence_after_sync();
                    // scales of this stage: four instructions' worth per weight tile and for the token tile
#pragma unroll
                    for (int j = 0; j < KSTEPS; ++j) {
#pragma unroll
                        for (int a = 0; a < NA; ++a)
                            tc::cp_sf_32x128b(tmem_sf + a * 16 + j * 4, tc::smem_desc_rows16(tc::smem_u32(sSFA(s, a)) + j * 512));
                        tc::cp_sf_32x128b(tmem_sf + NA * 16 + j * 4, tc::smem_desc_rows16(tc::smem_u32(sSFB(s)) + j * 512));
                    }
#pragma unroll
                    for (int j = 0; j < KSTEPS; ++j) {
                        const uint64_t bd = tc::smem_desc_sw128(tc::smem_u32(sB(s)) + j * 32);
#pragma unroll
                        for (int a = 0; a < NA; ++a) {
                            const uint64_t ad = tc::smem_desc_sw128(tc::smem_u32(sA(s, a)) + j * 32);
                            tc::mma_nvf4_ss(d_tmem + a * BN, ad, bd, idesc, tmem_sf + a * 16 + j * 4, tmem_sf + NA * 16 + j * 4,
                                            (kb > 0 || j > 0) ? 1u : 0u);
                        }
                    }
                    tc::mma_commit(&empty[s]);
                }
                if (ok) tc::mma_commit(&tmem_full[buf]);
            }
        }
    } else {
        const int q = warp & 3;               // TMEM lane quarter of this warp
        const int chunk_half = (warp - 2) >> 2; // which of the quarter's warps: it takes the 32-column chunk of that index
        // Everything the epilogue of a tile reads from global memory (its table entry, the weights' global scales, the
        // token rows' global scales) is fetched one tile ahead, while the previous tile is being stored: with a short
        // reduction (one or two stages per tile) those dependent loads would otherwise be the tile's critical path.
        struct Pre { Fp4Tile t; float ga, gu; float gb[BN / 32]; unsigned long long dst[BN / 32]; };
        auto prefetch = [&](int tile, Pre& pre) {
            pre.t = p.tiles[tile];
            const float* ga_p = pre.t.group < 0 ? p.gA2 : p.gA + (PAIR ? 2 : 1) * pre.t.group;
            pre.ga = __ldg(ga_p);
            pre.gu = PAIR ? __ldg(ga_p + 1) : 0.f;
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) {
                const bool in = c * 32 + lane < pre.t.b_valid;
                pre.gb[c] = in ? __ldg(p.gB + pre.t.b_row0 + c * 32 + lane) : 0.f;
                pre.dst[c] = 0ull;
                if (p.row_meta != nullptr && in) {
                    const int2 mt = __ldg(p.row_meta + pre.t.b_row0 + c * 32 + lane);
                    pre.dst[c] = (unsigned long long)(p.scatter_base[mt.x & 7] + (size_t)mt.y * p.ldo);
                } else if (p.col_rows != nullptr && in) {
                    const int row = __ldg(p.col_rows + pre.t.tab0 + c * 32 + lane);
                    if (row >= 0) pre.dst[c] = (unsigned long long)((char*)p.out + (size_t)row * p.ldo * (p.out_kind == 1 ? 4 : 2));
                }
            }
        };
        Pre cur;
        if ((int)blockIdx.x < total) prefetch(blockIdx.x, cur);
        int lt = 0;
        for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++lt) {
            const int buf = NBUF == 2 ? (lt & 1) : 0;
            const uint32_t par = NBUF == 2 ? ((lt >> 1) & 1) : (lt & 1);
            Pre nxt = cur;
            if (tile + (int)gridDim.x < total) prefetch(tile + gridDim.x, nxt);
            if (!tc::mbar_wait(&tmem_full[buf], par)) {
                if (lane == 0) atomicExch(p.err, 13);
                break;
            }
            tc::fence_after_sync();
            const Fp4Tile& t = cur.t;
            const int n = t.out_n0 + q * 32 + lane;                      // output column = weight row of this lane
            const uint32_t t_acc = tmem_base + ((uint32_t)(q * 32) << 16) + buf * Cfg::ACC_COLS;
            const float ga = cur.ga, gu = cur.gu;
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) {
                const int c0 = c * 32;
                if (c == chunk_half && c0 < t.b_valid) {                 // (uniform over the warp)
                    const float my_gb = cur.gb[c];                       // lane i holds token c0 + i's global scale
                    uint32_t r0[32], r1[32];
                    tc::tmem_ld_32x32(t_acc + c0, r0);
                    if (PAIR) tc::tmem_ld_32x32(t_acc + BN + c0, r1);
                    tc::tmem_ld_wait();
                    const int lim = min(32, t.b_valid - c0);
                    if (p.col_rows != nullptr) {
                        const unsigned long long my_dst = cur.dst[c];    // lane i holds where token column c0 + i goes (0: nowhere)
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float gb = __shfl_sync(0xffffffffu, my_gb, i);
                            const unsigned long long row = __shfl_sync(0xffffffffu, my_dst, i);
                            float v = __uint_as_float(r0[i]) * ga * gb;
                            if (PAIR) {
                                const float u = __uint_as_float(r1[i]) * gu * gb;
                                v = v / (1.f + __expf(-v)) * u;
                            }
                            if (i < lim && row != 0ull) {
                                if (p.out_kind == 1) reinterpret_cast<float*>(row)[n] = v;
                                else reinterpret_cast<bf16*>(row)[n] = __float2bfloat16(v);
                            }
                        }
                    } else if (p.out_kind == 1) {
                        float* dst = (float*)p.out + (size_t)(t.b_row0 + c0) * p.ldo + n;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float gb = __shfl_sync(0xffffffffu, my_gb, i);
                            float v = __uint_as_float(r0[i]) * ga * gb;
                            if (PAIR) {
                                const float u = __uint_as_float(r1[i]) * gu * gb;
                                v = v / (1.f + __expf(-v)) * u;
                            }
                            if (i < lim) dst[(size_t)i * p.ldo] = v;
                        }
                    } else if (p.row_meta != nullptr) {
                        const unsigned long long my_dst = cur.dst[c];    // lane i holds where token c0 + i's row goes
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float gb = __shfl_sync(0xffffffffu, my_gb, i);
                            bf16* row = reinterpret_cast<bf16*>(__shfl_sync(0xffffffffu, my_dst, i));
                            float v = __uint_as_float(r0[i]) * ga * gb;
                            if (PAIR) {
                                const float u = __uint_as_float(r1[i]) * gu * gb;
                                v = v / (1.f + __expf(-v)) * u;
                            }
                            if (i < lim) row[n] = __float2bfloat16(v);
                        }
                    } else {
                        bf16* dst = (bf16*)p.out + (size_t)(t.b_row0 + c0) * p.ldo + n;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float gb = __shfl_sync(0xffffffffu, my_gb, i);
                            float v = __uint_as_float(r0[i]) * ga * gb;
                            if (PAIR) {
                                const float u = __uint_as_float(r1[i]) * gu * gb;
                                v = v / (1.f + __expf(-v)) * u;
                            }
                            if (i < lim) dst[(size_t)i * p.ldo] = __float2bfloat16(v);
                        }
                    }
                }
            }
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&tmem_empty[buf]);
            cur = nxt;
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

int fp4_sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int BN, int PAIR>
int launch_fp4(const void* W, int w_rows, const void* X, int x_rows, const Fp4Params& p, int max_tiles, cudaStream_t s,
               const void* W2 = nullptr, int w2_rows = 0) {
    using Cfg = Fp4Cfg<BN, PAIR>;
    CUtensorMap tmA, tmB, tmA2;
    const uint64_t kb = (uint64_t)p.K / 2;
    int rc = make_tmap_2d(&tmA, W, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)w_rows, kb, kb, BM, BKB);
    if (rc) return rc;
    // tiles of a negative group read the second weight set; without one the map repeats the first (never used)
    rc = make_tmap_2d(&tmA2, W2 ? W2 : W, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)(W2 ? w2_rows : w_rows), kb, kb, BM, BKB);
    if (rc) return rc;
    rc = make_tmap_2d(&tmB, X, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)x_rows, kb, kb, BN, BKB);
    if (rc) return rc;
    auto kern = gemm_fp4_kernel<BN, PAIR>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
        attr_set = true;
    }
    const int grid = std::min(max_tiles, fp4_sm_count());
    sl_launch(kern, grid, Cfg::THREADS, Cfg::SMEM, s, tmA, tmB, tmA2, p);
    return (int)cudaGetLastError();
}

// ---- group padding and tile tables --------------------------------------------------------------------------------------
// pad[g] = first padded row of group g when every group is rounded up to a multiple of bn rows; pad[groups] = their total.
__global__ void fp4_group_pad_kernel(int* __restrict__ pad, const int* __restrict__ offsets, int groups, int bn) {
    pdl_grid_sync();
    __shared__ int cnt[1025];
    const int g = threadIdx.x;
    if (g < groups) cnt[g + 1] = (offsets[g + 1] - offsets[g] + bn - 1) / bn * bn;
    if (g == 0) cnt[0] = 0;
    __syncthreads();
    if (g == 0) for (int i = 1; i <= groups; ++i) cnt[i] += cnt[i - 1];
    __syncthreads();
    if (g <= groups) pad[g] = cnt[g];
}

// One block per group.  Group g owns token rows [offsets[g], offsets[g+1]) and weight rows [g * wrows, (g + 1) * wrows)
// (wrows = Nn, or 2 Nn for gate/up pairs with Nn output columns).  Tiles of a group: token blocks outermost.
__global__ void __launch_bounds__(256) fp4_build_tiles_kernel(Fp4Tile* __restrict__ tiles, int* __restrict__ num_tiles, const int* __restrict__ offsets,
                                                               const int* __restrict__ pad, int groups, int Nn, int pair, int bn, int max_tiles) {
    pdl_grid_sync();
    const int g = blockIdx.x;
    const int mt = Nn / BM;
    const int wrows = pair ? 2 * Nn : Nn;
    // tiles before this group = (padded rows before it / bn) * mt
    const int base = pad[g] / bn * mt;
    const int r0 = offsets[g], r1 = offsets[g + 1];
    const int nb = (r1 - r0 + bn - 1) / bn;
    for (int i = threadIdx.x; i < nb * mt; i += blockDim.x) {
        const int b = i / mt, m = i % mt;
        const int at = base + i;
        if (at < max_tiles) {
            Fp4Tile t;
            t.a_row0 = g * wrows + m * BM;
            t.sfa_blk0 = g * (wrows / BM) + m;
            t.b_row0 = r0 + b * bn;
            t.b_valid = min(bn, r1 - t.b_row0);
            t.out_n0 = m * BM;
            t.group = g;
            t.sfb_tile = pad[g] / bn + b;
            t.tab0 = 0;
            tiles[at] = t;
        }
    }
    if (g == groups - 1 && threadIdx.x == 0) *num_tiles = min(pad[groups] / bn * mt, max_tiles);
}

// ---- scale-factor tiles ------------------------------------------------------------------------------------------------
// Row-major e4m3 scales [mats][rows][kb] -> [mats][rows / 128][kb / 4][512] tiles (rows % 128 == 0, kb % 4 == 0).
__global__ void sf_tiles_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, size_t total_words, int rows, int kb) {
    pdl_grid_sync();
    // one thread moves the four scales of one (row, 64-index tile): a 32-bit word
    const int kt_n = kb / 4;
    for (size_t w = (size_t)blockIdx.x * blockDim.x + threadIdx.x; w < total_words; w += (size_t)gridDim.x * blockDim.x) {
        const size_t row_all = w / kt_n;
        const int kt = (int)(w % kt_n);
        const size_t mat = row_all / rows;
        const int r = (int)(row_all % rows);
        const uint32_t v = *reinterpret_cast<const uint32_t*>(src + row_all * kb + (size_t)kt * 4);
        const size_t blk = mat * (rows / 128) + r / 128;
        const int rr = r % 128;
        *reinterpret_cast<uint32_t*>(dst + (blk * kt_n + kt) * 512 + (rr % 32) * 16 + (rr / 32) * 4) = v;
    }
}

// ---- activation quantisation --------------------------------------------------------------------------------------------
// One block per output row, one thread per 64 consecutive values (one instruction's worth of the reduction): out row m =
// NVFP4 of x[src[m]] (or x[m]); per-row global scale g = amax / (6 * 448), block scale = e4m3(amax_16 / (6 g)), code =
// e2m1(x / (scale * g)).  With `terms` > 1 row m + j * rows holds the j-th residual (what the first j terms left over),
// quantised the same way.  Rows whose source is outside x are zero.  Scales go to tile (p / bn, k / 64), row p % bn, of
// the padded row p (see the file header); without groups p is the output row itself.
struct QuantParams {
    uint8_t* q; uint8_t* sf; float* g;
    const bf16* x; const int* src;
    int rows, x_rows, K, ldx, terms;
    const int* offsets; const int* pad; int groups, bn;
    const int* num_rows;           // optional: rows at or beyond *num_rows are skipped (receive buffers with spare capacity)
};

__device__ __forceinline__ float e2m1_value(uint32_t code) {
    const uint32_t m = code & 7u;
    // 0, .5, 1, 1.5, 2, 3, 4, 6
    const float mag = m < 2u ? 0.5f * (float)m : __uint_as_float(((m >> 1) + 126u) << 23) * ((m & 1u) ? 1.5f : 1.f);
    return (code & 8u) ? -mag : mag;
}

// `lpr` = 0: one block per row (one thread per 64 values).  Short rows (at most 2048 values) take `lpr` in {4, 8, 16, 32}
// lanes per row and 256 / lpr rows per block instead: a block per 256-value row would run four threads of a warp.
__global__ void __launch_bounds__(256) nvfp4_quantize_rows_kernel(const QuantParams p, int lpr, int launch_rows) {
    pdl_grid_sync();
    __shared__ float scratch[33];
    const int m = lpr ? blockIdx.x * (256 / lpr) + (int)threadIdx.x / lpr : (int)blockIdx.x;
    const int ks = lpr ? (int)threadIdx.x % lpr : (int)threadIdx.x;
    if (m >= launch_rows) return;
    if (p.num_rows != nullptr && m >= __ldg(p.num_rows)) return;
    const int KT = p.K / 64;
    if (m >= p.rows) {                             // padding rows of the last scale tile (ungrouped, one term): zero scales
        if (ks < KT) {
            const int tile = m / p.bn, r = m % p.bn;
            uint8_t* dst = p.sf + ((size_t)tile * KT + ks) * 512 + (r % 32) * 16;
            if (p.bn == 32) *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
            else *reinterpret_cast<uint32_t*>(dst + (r / 32) * 4) = 0u;
        }
        return;
    }
    const int sr = p.src ? p.src[m] : m;
    const bool valid = sr >= 0 && sr < p.x_rows && ks < KT;
    float v[64];
    if (valid) {
        const uint4* row = reinterpret_cast<const uint4*>(p.x + (size_t)sr * p.ldx + (size_t)ks * 64);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint4 w = __ldg(row + u);
            const float2 a = bf162_to_f2(w.x), b = bf162_to_f2(w.y), c = bf162_to_f2(w.z), d = bf162_to_f2(w.w);
            v[8 * u + 0] = a.x; v[8 * u + 1] = a.y; v[8 * u + 2] = b.x; v[8 * u + 3] = b.y;
            v[8 * u + 4] = c.x; v[8 * u + 5] = c.y; v[8 * u + 6] = d.x; v[8 * u + 7] = d.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) v[i] = 0.f;
    }
    // padded row of the scales
    int prow0 = m;
    if (p.offsets != nullptr) {
        int lo = 0, hi = p.groups;                 // last group whose first row is <= m
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (__ldg(p.offsets + mid) <= m) lo = mid; else hi = mid;
        }
        prow0 = __ldg(p.pad + lo) + (m - __ldg(p.offsets + lo));
    }
    for (int term = 0; term < p.terms; ++term) {
        const size_t orow = (size_t)m + (size_t)term * p.rows;
        const int prow = p.offsets != nullptr ? prow0 : (int)orow;
        float bm[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            float a = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) a = fmaxf(a, fabsf(v[16 * b + i]));
            bm[b] = a;
        }
        float amax = fmaxf(fmaxf(bm[0], bm[1]), fmaxf(bm[2], bm[3]));
        if (lpr) {                                 // the row's lanes are an aligned group of one warp
            const unsigned lane = threadIdx.x & 31u;
            const unsigned gmask = (lpr == 32 ? 0xffffffffu : ((1u << lpr) - 1u)) << (lane & ~(unsigned)(lpr - 1));
            for (int o = lpr >> 1; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, o));
        } else {
            amax = block_max(amax, scratch);
        }
        const float gs = amax > 0.f ? amax / (6.f * 448.f) : 1.f;
        if (ks == 0) p.g[orow] = gs;
        if (ks < KT) {
            const float inv_g = 1.f / gs;
            uint32_t sc_word = 0, packed[8];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint8_t sc8 = float_to_e4m3(bm[b] * inv_g * (1.f / 6.f));
                sc_word |= (uint32_t)sc8 << (8 * b);
                const float dq = e4m3_to_float(sc8) * gs;               // value of code 1.0
                const float inv = dq > 0.f ? 1.f / dq : 0.f;
                uint32_t w0 = 0, w1 = 0;
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    uint32_t two;
                    // the first source of the conversion lands in the high nibble
                    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u32.u8 %0, t; }"
                        : "=r"(two) : "f"(v[16 * b + i + 1] * inv), "f"(v[16 * b + i] * inv));
                    if (i < 8) w0 |= two << (4 * i); else w1 |= two << (4 * (i - 8));
                    if (p.terms > 1) {                                   // what this term represents comes off the remainder
                        v[16 * b + i] -= e2m1_value(two & 0xFu) * dq;
                        v[16 * b + i + 1] -= e2m1_value(two >> 4) * dq;
                    }
                }
                packed[2 * b] = w0; packed[2 * b + 1] = w1;
            }
            uint4* qd = reinterpret_cast<uint4*>(p.q + orow * (size_t)(p.K / 2) + (size_t)ks * 32);
            qd[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            qd[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            const int tile = prow / p.bn, r = prow % p.bn;
            uint8_t* dst = p.sf + ((size_t)tile * KT + ks) * 512 + (r % 32) * 16;
            // 32-row tiles use the first of the four words of a 16-byte piece; the other three are written too (zero), so
            // the whole piece is defined without a separate clear
            if (p.bn == 32) *reinterpret_cast<uint4*>(dst) = make_uint4(sc_word, 0u, 0u, 0u);
            else *reinterpret_cast<uint32_t*>(dst + (r / 32) * 4) = sc_word;
        }
    }
}

// Quantised rows gathered into another order without quantising them again: out row m = source row src[m] (codes,
// global scale, and the scale words moved from the source's tile layout, one group of `src_bn`-row tiles, to the padded
// rows of `offsets` / `pad`).  One block per output row, one thread per 64 reduction indices.
struct GatherParams {
    uint8_t* q; uint8_t* sf; float* g;
    const uint8_t* q_src; const uint8_t* sf_src; const float* g_src; const int* src;
    int rows, src_rows, K, src_bn;
    const int* offsets; const int* pad; int groups, bn;
};

__global__ void __launch_bounds__(256) nvfp4_gather_rows_kernel(const GatherParams p) {
    pdl_grid_sync();
    const int m = blockIdx.x, ks = threadIdx.x;
    const int KT = p.K / 64;
    if (ks >= KT) return;
    const int sr = p.src[m];
    const bool valid = sr >= 0 && sr < p.src_rows;
    int lo = 0, hi = p.groups;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(p.offsets + mid) <= m) lo = mid; else hi = mid;
    }
    const int prow = __ldg(p.pad + lo) + (m - __ldg(p.offsets + lo));
    uint4 c0 = make_uint4(0, 0, 0, 0), c1 = c0;
    uint32_t sc = 0;
    if (valid) {
        const uint4* qs = reinterpret_cast<const uint4*>(p.q_src + (size_t)sr * (p.K / 2) + (size_t)ks * 32);
        c0 = __ldg(qs); c1 = __ldg(qs + 1);
        const int st = sr / p.src_bn, r = sr % p.src_bn;
        sc = __ldg(reinterpret_cast<const uint32_t*>(p.sf_src + ((size_t)st * KT + ks) * 512 + (r % 32) * 16 + (r / 32) * 4));
    }
    uint4* qd = reinterpret_cast<uint4*>(p.q + (size_t)m * (p.K / 2) + (size_t)ks * 32);
    qd[0] = c0; qd[1] = c1;
    const int tile = prow / p.bn, r = prow % p.bn;
    *reinterpret_cast<uint32_t*>(p.sf + ((size_t)tile * KT + ks) * 512 + (r % 32) * 16 + (r / 32) * 4) = sc;
    if (ks == 0) p.g[m] = valid ? __ldg(p.g_src + sr) : 1.f;
}

template <int PAIR>
int dispatch_bn(int bn, const void* W, int w_rows, const void* X, int x_rows, const Fp4Params& p, int max_tiles, cudaStream_t s,
                const void* W2 = nullptr, int w2_rows = 0) {
    switch (bn) {
        case 32: return launch_fp4<32, PAIR>(W, w_rows, X, x_rows, p, max_tiles, s, W2, w2_rows);
        case 64: return launch_fp4<64, PAIR>(W, w_rows, X, x_rows, p, max_tiles, s, W2, w2_rows);
        case 128: return launch_fp4<128, PAIR>(W, w_rows, X, x_rows, p, max_tiles, s, W2, w2_rows);
        default: return -1;
    }
}

// ---- decode-time MoE: plan and tile tables for up to 32 token rows ---------------------------------------------------------
// Every expert that some token chose gets a slot (in order of its first route); slot s owns rows [32 s, 32 s + 32) of the
// activation buffer, one per token routed to it (in token order).  The shared expert, if any, takes the slot after the
// last routed one with all T tokens.
//   gate/up GEMM  tiles {slot, 128-row block of I}: token operand = ALL T token rows (the same for every tile);
//                 tab1[32 s + t] = 32 s + (rank of token t among the slot's tokens), or -1 if t did not choose it
//   down GEMM     tiles {slot, 128-row block of H}: token operand = the slot's 32 activation rows;
//                 tab2[32 s + j] = route of the slot's j-th token (t * top_k + choice; T * top_k + t for the shared expert)
// so neither GEMM needs its rows sorted or gathered: the first drops the columns a slot does not own, the second scatters
// its columns back to per-route rows.  One block of 256 threads; `sh` = 10 E + 16 ints.
struct Fp4DecodePlan {
    const int* ids;                 // [T, top_k] expert ids
    int T, top_k, expert_offset, num_local, has_shared;
    int I, H;                       // expert intermediate / hidden size (multiples of 128)
    Fp4Tile* tiles1; int* ntiles1;  // gate/up tiles, at most (max_slots + 1) * I / 128
    Fp4Tile* tiles2; int* ntiles2;  // down tiles, at most (max_slots + 1) * H / 128
    int* tab1; int* tab2;           // [(max_slots + 1) * 32]
    int* num_rows;                  // activation rows in use: 32 * slots
    int max_slots;
};

__global__ void __launch_bounds__(256) fp4_decode_plan_kernel(const Fp4DecodePlan p) {
    pdl_grid_sync();
    extern __shared__ int sh[];
    const int E = p.num_local, n = p.T * p.top_k;
    int* cnt = sh;                                 // [8][E] routes of expert e in warp w of the current pass
    int* run = cnt + 8 * E;                        // [E] routes of expert e in earlier passes
    int* slot_of = run + E;                        // [E] slot of expert e (-1: untouched)
    __shared__ int s_slots;
    __shared__ int wcnt[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < 9 * E; i += 256) sh[i] = 0;
    for (int i = tid; i < E; i += 256) slot_of[i] = -1;
    for (int i = tid; i < (p.max_slots + 1) * 32; i += 256) { p.tab1[i] = -1; p.tab2[i] = -1; }
    if (tid == 0) s_slots = 0;
    __syncthreads();
    for (int base = 0; base < n; base += 256) {
        const int r = base + tid;
        int e = -1;
        if (r < n) {
            const int le = p.ids[r] - p.expert_offset;
            e = (le >= 0 && le < E) ? le : -1;
        }
        const unsigned same = __match_any_sync(0xffffffffu, e);
        const int rank_in_warp = __popc(same & ((1u << lane) - 1));
        if (e >= 0 && rank_in_warp == 0) cnt[warp * E + e] = __popc(same);
        __syncthreads();
        int before = -1;
        if (e >= 0) {
            before = run[e] + rank_in_warp;
            for (int w = 0; w < warp; ++w) before += cnt[w * E + e];
        }
        const bool first = before == 0;            // the expert's first route claims its slot, in route order
        const unsigned m = __ballot_sync(0xffffffffu, first);
        if (lane == 0) wcnt[warp] = __popc(m);
        __syncthreads();
        int slot = s_slots, total = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            if (w < warp) slot += wcnt[w];
            total += wcnt[w];
        }
        slot += __popc(m & ((1u << lane) - 1));
        if (first && slot < p.max_slots) slot_of[e] = slot;
        __syncthreads();
        if (before >= 0 && before < 32) {
            const int sl = slot_of[e];
            if (sl >= 0) {
                const int t = r / p.top_k;
                p.tab1[sl * 32 + t] = sl * 32 + before;
                p.tab2[sl * 32 + before] = r;
            }
        }
        if (tid == 0) s_slots = min(p.max_slots, s_slots + total);
        __syncthreads();
        for (int i = tid; i < E; i += 256) {
            int c = 0;
#pragma unroll
            for (int w = 0; w < 8; ++w) { c += cnt[w * E + i]; cnt[w * E + i] = 0; }
            run[i] += c;
        }
        __syncthreads();
    }
    const int slots = s_slots;
    const int all = slots + (p.has_shared ? 1 : 0);
    if (p.has_shared) {
        for (int t = tid; t < p.T; t += 256) {
            p.tab1[slots * 32 + t] = slots * 32 + t;
            p.tab2[slots * 32 + t] = n + t;
        }
    }
    const int mt1 = p.I / BM, mt2 = p.H / BM;
    // slot -> expert: the inverse of slot_of, built in shared memory on top of cnt (free by now)
    int* exp_of = cnt;
    for (int e = tid; e < E; e += 256)
        if (slot_of[e] >= 0) exp_of[slot_of[e]] = e;
    __syncthreads();
    for (int i = tid; i < all * mt1; i += 256) {
        const int sl = i / mt1, m = i % mt1;
        const bool shd = sl >= slots;
        const int e = shd ? 0 : exp_of[sl];
        Fp4Tile t;
        t.a_row0 = e * 2 * p.I + m * BM;           // gate rows; the up rows follow I rows later
        t.sfa_blk0 = e * (2 * p.I / BM) + m;
        t.b_row0 = 0;
        t.b_valid = p.T;
        t.out_n0 = m * BM;
        t.group = shd ? -1 : e;
        t.sfb_tile = 0;
        t.tab0 = sl * 32;
        p.tiles1[i] = t;
    }
    for (int i = tid; i < all * mt2; i += 256) {
        const int sl = i / mt2, m = i % mt2;
        const bool shd = sl >= slots;
        const int e = shd ? 0 : exp_of[sl];
        Fp4Tile t;
        t.a_row0 = e * p.H + m * BM;
        t.sfa_blk0 = e * (p.H / BM) + m;
        t.b_row0 = sl * 32;
        t.b_valid = shd ? p.T : min(32, run[e]);
        t.out_n0 = m * BM;
        t.group = shd ? -1 : e;
        t.sfb_tile = sl;
        t.tab0 = sl * 32;
        p.tiles2[i] = t;
    }
    if (tid == 0) {
        *p.ntiles1 = all * mt1;
        *p.ntiles2 = all * mt2;
        *p.num_rows = all * 32;
    }
}

}  // namespace

// Bytes per tile-table entry (the caller allocates max_tiles of them).
SL_API int sl_fp4_tile_bytes() { return (int)sizeof(Fp4Tile); }

// pad int32 [groups + 1]: first padded row of every group (groups rounded up to multiples of bn rows) and their total.
SL_API int sl_fp4_group_pad(void* pad, const void* offsets, int groups, int bn, cudaStream_t s) {
    if (groups <= 0 || groups > 1024 || (bn != 32 && bn != 64 && bn != 128)) return -1;
    sl_launch(fp4_group_pad_kernel, 1, 1024, 0, s, (int*)pad, (const int*)offsets, groups, bn);
    return (int)cudaGetLastError();
}

// Tile table of a grouped product: `offsets` int32 [groups + 1] on the device, `pad` from sl_fp4_group_pad with the
// same bn, Nn output columns per group (a multiple of 128), `pair` = gate/up weight stacks [groups][2 Nn][K/2] with
// the SiLU * mul epilogue.  At most (pad[groups] / bn) * (Nn / 128) tiles.
SL_API int sl_fp4_build_tiles(void* tiles, void* num_tiles, const void* offsets, const void* pad, int groups, int Nn, int pair, int bn,
                              int max_tiles, cudaStream_t s) {
    if (groups <= 0 || groups > 1024 || Nn % BM != 0 || (bn != 32 && bn != 64 && bn != 128)) return -1;
    sl_launch(fp4_build_tiles_kernel, groups, 256, 0, s, (Fp4Tile*)tiles, (int*)num_tiles, (const int*)offsets, (const int*)pad, groups, Nn,
              pair, bn, max_tiles);
    return (int)cudaGetLastError();
}

// Grouped (or, with one group, plain) NVFP4 x NVFP4 product over a tile table.
//   W [w_rows, K/2] packed weights, sfa their scale tiles, gA [groups] (pair: [groups][2]) fp32
//   X [x_rows, K/2] packed activation rows, sfb their scale tiles (padded rows, see the file header), gB [x_rows] fp32
//   out [x_rows, ldo] bf16 (out_kind 0) or fp32 (1); pair: out = silu(gate) * up with Nn = pair_rows output columns
// K % 256 == 0.  `err` is set to a non-zero site code when a bounded wait expired.
SL_API int sl_gemm_fp4_tcgen05(const void* W, const void* sfa, const void* gA, int w_rows, const void* X, const void* sfb, const void* gB,
                               int x_rows, void* out, int ldo, int out_kind, int K, int pair_rows, int bn, const void* tiles,
                               const void* num_tiles, int max_tiles, void* err, cudaStream_t s) {
    if (w_rows <= 0 || x_rows <= 0 || max_tiles <= 0) return 0;
    if (K % 256 != 0 || K <= 0 || pair_rows % BM != 0) return -1;
    Fp4Params p{};
    p.sfa = (const uint8_t*)sfa; p.sfb = (const uint8_t*)sfb; p.gA = (const float*)gA; p.gB = (const float*)gB; p.out = out; p.K = K;
    p.ldo = ldo; p.out_kind = out_kind; p.pair_rows = pair_rows; p.pair_blks = pair_rows / BM;
    p.tiles = (const Fp4Tile*)tiles; p.num_tiles = (const int*)num_tiles; p.err = (int*)err;
    return pair_rows > 0 ? dispatch_bn<1>(bn, W, w_rows, X, x_rows, p, max_tiles, s) : dispatch_bn<0>(bn, W, w_rows, X, x_rows, p, max_tiles, s);
}

// Plan + tile tables of the decode-time MoE layer on this kernel (see fp4_decode_plan_kernel).  T <= 32, T * top_k <= 512,
// num_local <= 1024; `max_slots` bounds the experts that can be touched (min(num_local, T * top_k)).
SL_API int sl_fp4_decode_plan(const void* ids, int T, int top_k, int expert_offset, int num_local, int has_shared, int I, int H,
                              void* tiles1, void* ntiles1, void* tiles2, void* ntiles2, void* tab1, void* tab2, void* num_rows,
                              int max_slots, cudaStream_t s) {
    if (T <= 0) return 0;
    if (T > 32 || T * top_k > 512 || num_local < 1 || num_local > 1024 || I % BM != 0 || H % BM != 0 || max_slots < 1) return -1;
    Fp4DecodePlan p{(const int*)ids, T, top_k, expert_offset, num_local, has_shared, I, H, (Fp4Tile*)tiles1, (int*)ntiles1,
                    (Fp4Tile*)tiles2, (int*)ntiles2, (int*)tab1, (int*)tab2, (int*)num_rows, max_slots};
    const size_t smem = (size_t)(10 * num_local + 16) * sizeof(int);
    if (smem > 48 * 1024) return -1;
    sl_launch(fp4_decode_plan_kernel, 1, 256, smem, s, p);
    return (int)cudaGetLastError();
}

// The product with the column-row table epilogue (decode MoE): token column c of a tile goes to output row
// col_rows[tile.tab0 + c] (bf16 or f32 rows of `ldo` elements; negative: dropped).  Tiles of a negative group take the
// second weight set (W2 / sfa2 / gA2: the shared expert).
SL_API int sl_gemm_fp4_tcgen05_tab(const void* W, const void* sfa, const void* gA, int w_rows, const void* W2, const void* sfa2,
                                   const void* gA2, int w2_rows, const void* X, const void* sfb, const void* gB, int x_rows,
                                   void* out, int ldo, int out_kind, const void* col_rows, int K, int pair_rows, int bn,
                                   const void* tiles, const void* num_tiles, int max_tiles, void* err, cudaStream_t s) {
    if (w_rows <= 0 || x_rows <= 0 || max_tiles <= 0) return 0;
    if (K % 256 != 0 || K <= 0 || pair_rows % BM != 0 || col_rows == nullptr || out == nullptr) return -1;
    Fp4Params p{};
    p.sfa = (const uint8_t*)sfa; p.sfb = (const uint8_t*)sfb; p.gA = (const float*)gA; p.gB = (const float*)gB; p.out = out; p.K = K;
    p.ldo = ldo; p.out_kind = out_kind; p.pair_rows = pair_rows; p.pair_blks = pair_rows / BM;
    p.tiles = (const Fp4Tile*)tiles; p.num_tiles = (const int*)num_tiles; p.err = (int*)err;
    p.col_rows = (const int*)col_rows;
    p.sfa2 = (const uint8_t*)(sfa2 ? sfa2 : sfa); p.gA2 = (const float*)(gA2 ? gA2 : gA);
    return pair_rows > 0 ? dispatch_bn<1>(bn, W, w_rows, X, x_rows, p, max_tiles, s, W2, w2_rows)
                         : dispatch_bn<0>(bn, W, w_rows, X, x_rows, p, max_tiles, s, W2, w2_rows);
}

// The same product with the expert-parallel combine epilogue: bf16 output row m goes to
// scatter_base[row_meta[m].x] + row_meta[m].y * ldo (`scatter_base`: W pointers, peer mappings of the home ranks'
// combine buffers).
SL_API int sl_gemm_fp4_tcgen05_scatter(const void* W, const void* sfa, const void* gA, int w_rows, const void* X, const void* sfb,
                                       const void* gB, int x_rows, const void* row_meta, void* const* scatter_base, int world, int ldo,
                                       int K, int bn, const void* tiles, const void* num_tiles, int max_tiles, void* err,
                                       cudaStream_t s) {
    if (w_rows <= 0 || x_rows <= 0 || max_tiles <= 0) return 0;
    if (K % 256 != 0 || K <= 0 || row_meta == nullptr || world < 1 || world > 8) return -1;
    Fp4Params p{};
    p.sfa = (const uint8_t*)sfa; p.sfb = (const uint8_t*)sfb; p.gA = (const float*)gA; p.gB = (const float*)gB; p.out = nullptr; p.K = K;
    p.ldo = ldo; p.out_kind = 0; p.pair_rows = 0; p.pair_blks = 0;
    p.tiles = (const Fp4Tile*)tiles; p.num_tiles = (const int*)num_tiles; p.err = (int*)err;
    p.row_meta = (const int2*)row_meta;
    for (int r = 0; r < 8; ++r) p.scatter_base[r] = (bf16*)scatter_base[r < world ? r : 0];
    return dispatch_bn<0>(bn, W, w_rows, X, x_rows, p, max_tiles, s);
}

// Row-major block scales [mats][rows][K/16] -> the tile layout the kernel above loads (rows % 128 == 0, K % 64 == 0).
SL_API int sl_nvfp4_sf_tiles(void* dst, const void* src, int mats, int rows, int K, cudaStream_t s) {
    if (mats <= 0 || rows <= 0) return 0;
    if (rows % 128 != 0 || K % 64 != 0) return -1;
    const size_t words = (size_t)mats * rows * (K / 64);
    const int blocks = (int)std::min<size_t>((words + 255) / 256, 148 * 16);
    sl_launch(sf_tiles_kernel, blocks, 256, 0, s, (uint8_t*)dst, (const uint8_t*)src, words, rows, K / 16);
    return (int)cudaGetLastError();
}

// Already quantised rows (q_src / sf_src / g_src: `src_rows` ungrouped rows whose scale tiles were written for `src_bn`-row
// tiles) gathered into grouped order: out row m = source row src[m], scales placed by `offsets` / `pad` / `bn`.
SL_API int sl_nvfp4_gather_rows(void* q, void* sf, void* g, const void* q_src, const void* sf_src, const void* g_src, const void* src,
                                int rows, int src_rows, int K, int src_bn, const void* offsets, const void* pad, int groups, int bn,
                                cudaStream_t s) {
    if (rows <= 0) return 0;
    if (K % 64 != 0 || K > 16384 || src == nullptr || offsets == nullptr || pad == nullptr) return -1;
    GatherParams p{(uint8_t*)q, (uint8_t*)sf, (float*)g, (const uint8_t*)q_src, (const uint8_t*)sf_src, (const float*)g_src,
                   (const int*)src, rows, src_rows, K, src_bn, (const int*)offsets, (const int*)pad, groups, bn};
    sl_launch(nvfp4_gather_rows_kernel, rows, (K / 64 + 31) / 32 * 32, 0, s, p);
    return (int)cudaGetLastError();
}

// bf16 rows -> NVFP4 rows (+ residual terms).  q [rows * terms, K/2], g [rows * terms], sf = scale tiles
// [padded rows / bn][K/64][512]; `src` (int32 [rows], may be null) gathers: output row m quantises x[src[m]].
// `offsets` / `pad` (may be null: one group, no padding) place the scales of grouped rows, see sl_fp4_group_pad;
// `num_rows` (device int, may be null) limits the rows that are really quantised.  Without groups and with one term the
// scale tiles need no clearing by the caller (padding rows of the last tile are zeroed here); otherwise pass them zeroed.
// K % 64 == 0, K <= 16384, ldx % 8 == 0, x 16-byte aligned.
SL_API int sl_nvfp4_quantize_rows(void* q, void* sf, void* g, const void* x, const void* src, int rows, int x_rows, int K, int ldx,
                                  int terms, const void* offsets, const void* pad, int groups, int bn, const void* num_rows,
                                  cudaStream_t s) {
    if (rows <= 0) return 0;
    if (K % 64 != 0 || K > 16384 || terms < 1 || terms > 4 || ldx % 8 != 0 || ((uintptr_t)x & 15) != 0) return -1;
    if (bn != 32 && bn != 64 && bn != 128) return -1;
    if ((offsets != nullptr) != (pad != nullptr) || (offsets != nullptr && terms != 1)) return -1;
    QuantParams p{(uint8_t*)q, (uint8_t*)sf, (float*)g, (const bf16*)x, (const int*)src, rows, x_rows, K, ldx, terms,
                  (const int*)offsets, (const int*)pad, groups, bn, (const int*)num_rows};
    const int threads = (K / 64 + 31) / 32 * 32;
    // ungrouped rows of one term: the blocks past `rows` zero the scales of the last tile's padding rows, so the caller
    // need not clear the scale tiles first
    const int launch_rows = (offsets == nullptr && terms == 1) ? (rows + bn - 1) / bn * bn : rows;
    if (K <= 2048) {
        int lpr = 4;
        while (lpr * 64 < K) lpr <<= 1;
        const int rpb = 256 / lpr;
        sl_launch(nvfp4_quantize_rows_kernel, (launch_rows + rpb - 1) / rpb, 256, 0, s, p, lpr, launch_rows);
    } else {
        sl_launch(nvfp4_quantize_rows_kernel, launch_rows, threads, 0, s, p, 0, launch_rows);
    }
    return (int)cudaGetLastError();
}
