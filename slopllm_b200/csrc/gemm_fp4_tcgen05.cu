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
//   W   packed codes [rows, K/2] (two per byte, even index in the low nibble), TMA-tiled with the 128-byte swizzle
//   SFA weight scales re-laid once at load time into 512-byte tiles of 128 rows x 4 scales (the layout `tcgen05.cp`
//       broadcasts into TMEM): byte (r % 32) * 16 + (r / 32) * 4 + (kb % 4) of tile (r / 128, kb / 4), see sl_nvfp4_sf_tiles
//   X   packed codes [tokens, K/2] written by sl_nvfp4_quantize_rows, gB[tokens] fp32, scales as [K/64][tokens][16 bytes]:
//       the four scales of one token and one instruction (64 indices) in the first four bytes of a 16-byte row.  Token
//       rows may start anywhere: each 32-token group is its own N = 32 instruction, and 32 such rows are exactly what one
//       `tcgen05.cp` moves (scale columns in TMEM stay 4-column aligned)
//
// Warp roles (192 threads): warp 0 issues TMA / bulk copies into a multi-stage ring, warp 1 copies scales into TMEM and
// issues the MMAs, warps 2-5 read the accumulators out of TMEM (one lane = one weight row) and store the transposed
// tile.  Two accumulator buffers when TMEM allows, so a tile's epilogue overlaps the next tile's MMAs.  No cluster
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
    int a_row0, a_row1;            // first weight row of the tile (and of the paired "up" tile, -1: none)
    int sfa_blk0, sfa_blk1;        // 128-row scale blocks of those rows
    int b_row0, b_valid;           // first token row, number of valid token rows (<= BN)
    int out_n0, group;             // output column of weight row 0 of the tile, group (expert) for the global scales
};

template <int BN, int PAIR>
struct Fp4Cfg {
    static constexpr int NA = PAIR ? 2 : 1;
    static constexpr int A_BYTES = BM * BKB, SFA_BYTES = 2048, B_BYTES = BN * BKB, SFB_BYTES = KSTEPS * BN * 16;
    static constexpr int TX = NA * (A_BYTES + SFA_BYTES) + B_BYTES + SFB_BYTES;      // bytes that land per stage
    static constexpr int STAGE = (TX + 1023) / 1024 * 1024;
    static constexpr int STAGES = (200 * 1024) / STAGE > 8 ? 8 : (200 * 1024) / STAGE;
    static constexpr int SMEM = STAGES * STAGE + 1024 + 256;
    static constexpr int ACC_COLS = NA * BN;
    static constexpr int SF_COLS = NA * 16 + (BN / 32) * 16;
    static constexpr int NBUF = (2 * ACC_COLS + SF_COLS <= 512) ? 2 : 1;
    static constexpr int TMEM_COLS = (NBUF * ACC_COLS + SF_COLS <= 64) ? 64 : (NBUF * ACC_COLS + SF_COLS <= 128) ? 128
                                     : (NBUF * ACC_COLS + SF_COLS <= 256) ? 256 : 512;
};

struct Fp4Params {
    const uint8_t* sfa;            // scale tiles [blocks][K/64][512]
    const float* gA;               // [groups] or [groups][2] (PAIR: gate, up) global scales of the weights
    const float* gB;               // [tokens] global scales of the activation rows
    void* out;                     // [tokens, ldo]: bf16 / f32 (out_kind 0 / 1)
    int K, ldo, out_kind;
    const Fp4Tile* tiles; const int* num_tiles;
    int* err;
};

template <int BN, int PAIR>
__global__ void __launch_bounds__(192) gemm_fp4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                                       const __grid_constant__ CUtensorMap tmSFB, const Fp4Params p) {
    using Cfg = Fp4Cfg<BN, PAIR>;
    constexpr int STAGES = Cfg::STAGES, NA = Cfg::NA, NBUF = Cfg::NBUF;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // stage layout: A tiles (1024-aligned) | B tile | SFA tiles | SFB rows
    auto sA = [&](int s, int a) { return smem + (size_t)s * Cfg::STAGE + (size_t)a * Cfg::A_BYTES; };
    auto sB = [&](int s) { return smem + (size_t)s * Cfg::STAGE + (size_t)NA * Cfg::A_BYTES; };
    auto sSFA = [&](int s, int a) { return smem + (size_t)s * Cfg::STAGE + (size_t)NA * Cfg::A_BYTES + Cfg::B_BYTES + (size_t)a * Cfg::SFA_BYTES; };
    auto sSFB = [&](int s) { return smem + (size_t)s * Cfg::STAGE + (size_t)NA * (Cfg::A_BYTES + Cfg::SFA_BYTES) + Cfg::B_BYTES; };
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
        tc::tma_prefetch_desc(&tmSFB);
        for (int s = 0; s < STAGES; ++s) { tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { tc::mbar_init(&tmem_full[b], 1); tc::mbar_init(&tmem_empty[b], 4); }
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
    const uint32_t tmem_sf = tmem_base + NBUF * Cfg::ACC_COLS;          // SFA: NA x 16 columns, then SFB: (BN/32) x 16
    pdl_grid_sync();

    const int total = *p.num_tiles;
    const int num_kb = p.K / (2 * BKB);
    const int KT = p.K / 64;                                            // scale tiles of 4 scales along K

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
                const Fp4Tile t = p.tiles[tile];
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!tc::mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1)) { atomicExch(p.err, 11); ok = false; break; }
                    tc::mbar_expect_tx(&full[s], Cfg::TX);
                    tc::tma_load_2d(sA(s, 0), &tmA, &full[s], kb * BKB, t.a_row0);
                    tc::bulk_load_1d(sSFA(s, 0), p.sfa + ((size_t)t.sfa_blk0 * KT + (size_t)kb * KSTEPS) * 512, Cfg::SFA_BYTES, &full[s]);
                    if (PAIR) {
                        tc::tma_load_2d(sA(s, 1), &tmA, &full[s], kb * BKB, t.a_row1);
                        tc::bulk_load_1d(sSFA(s, 1), p.sfa + ((size_t)t.sfa_blk1 * KT + (size_t)kb * KSTEPS) * 512, Cfg::SFA_BYTES, &full[s]);
                    }
                    tc::tma_load_2d(sB(s), &tmB, &full[s], kb * BKB, t.b_row0);
                    tc::tma_load_3d(sSFB(s), &tmSFB, &full[s], 0, t.b_row0, kb * KSTEPS);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = tc::idesc_nvf4(BM, 32);
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
                    // scales of this stage: 4 instructions' worth per weight tile, 4 per 32-token group
#pragma unroll
                    for (int a = 0; a < NA; ++a)
#pragma unroll
                        for (int j = 0; j < KSTEPS; ++j)
                            tc::cp_sf_32x128b(tmem_sf + a * 16 + j * 4, tc::smem_desc_rows16(tc::smem_u32(sSFA(s, a)) + j * 512));
#pragma unroll
                    for (int q = 0; q < BN / 32; ++q)
#pragma unroll
                        for (int j = 0; j < KSTEPS; ++j)
                            tc::cp_sf_32x128b(tmem_sf + NA * 16 + (q * KSTEPS + j) * 4,
                                              tc::smem_desc_rows16(tc::smem_u32(sSFB(s)) + (j * BN + q * 32) * 16));
#pragma unroll
                    for (int j = 0; j < KSTEPS; ++j) {
#pragma unroll
                        for (int a = 0; a < NA; ++a) {
                            const uint64_t ad = tc::smem_desc_sw128(tc::smem_u32(sA(s, a)) + j * 32);
#pragma unroll
                            for (int q = 0; q < BN / 32; ++q) {
                                const uint64_t bd = tc::smem_desc_sw128(tc::smem_u32(sB(s)) + q * 4096 + j * 32);
                                tc::mma_nvf4_ss(d_tmem + a * BN + q * 32, ad, bd, idesc, tmem_sf + a * 16 + j * 4, tmem_sf + NA * 16 + (q * KSTEPS + j) * 4,
                                                (kb > 0 || j > 0) ? 1u : 0u);
                            }
                        }
                    }
                    tc::mma_commit(&empty[s]);
                }
                if (ok) tc::mma_commit(&tmem_full[buf]);
            }
        }
    } else {
        const int q = warp & 3;               // TMEM lane quarter of this warp
        int lt = 0;
        for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++lt) {
            const int buf = NBUF == 2 ? (lt & 1) : 0;
            const uint32_t par = NBUF == 2 ? ((lt >> 1) & 1) : (lt & 1);
            if (!tc::mbar_wait(&tmem_full[buf], par)) {
                if (lane == 0) atomicExch(p.err, 13);
                break;
            }
            tc::fence_after_sync();
            const Fp4Tile t = p.tiles[tile];
            const int n = t.out_n0 + q * 32 + lane;                      // output column = weight row of this lane
            const uint32_t t_acc = tmem_base + ((uint32_t)(q * 32) << 16) + buf * Cfg::ACC_COLS;
            const float ga = PAIR ? p.gA[2 * t.group] : p.gA[t.group];
            const float gu = PAIR ? p.gA[2 * t.group + 1] : 0.f;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (c0 >= t.b_valid) break;
                uint32_t r0[32], r1[32];
                tc::tmem_ld_32x32(t_acc + c0, r0);
                if (PAIR) tc::tmem_ld_32x32(t_acc + BN + c0, r1);
                tc::tmem_ld_wait();
                for (int i = 0; i < 32 && c0 + i < t.b_valid; ++i) {
                    const int tok = t.b_row0 + c0 + i;
                    const float gb = p.gB[tok];
                    float v = __uint_as_float(r0[i]) * ga * gb;
                    if (PAIR) {
                        const float u = __uint_as_float(r1[i]) * gu * gb;
                        v = v / (1.f + __expf(-v)) * u;
                    }
                    if (p.out_kind == 1) ((float*)p.out)[(size_t)tok * p.ldo + n] = v;
                    else ((bf16*)p.out)[(size_t)tok * p.ldo + n] = __float2bfloat16(v);
                }
            }
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&tmem_empty[buf]);
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
int launch_fp4(const void* W, int w_rows, const void* X, int x_rows, const void* sfb, const Fp4Params& p, int max_tiles, cudaStream_t s) {
    using Cfg = Fp4Cfg<BN, PAIR>;
    CUtensorMap tmA, tmB, tmS;
    const uint64_t kb = (uint64_t)p.K / 2;
    int rc = make_tmap_2d(&tmA, W, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)w_rows, kb, kb, BM, BKB);
    if (rc) return rc;
    rc = make_tmap_2d(&tmB, X, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)x_rows, kb, kb, BN, BKB);
    if (rc) return rc;
    rc = make_tmap_3d_rows16(&tmS, sfb, (uint64_t)p.K / 64, (uint64_t)x_rows, KSTEPS, BN);
    if (rc) return rc;
    auto kern = gemm_fp4_kernel<BN, PAIR>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
        attr_set = true;
    }
    const int grid = std::min(max_tiles, fp4_sm_count());
    sl_launch(kern, grid, 192, Cfg::SMEM, s, tmA, tmB, tmS, p);
    return (int)cudaGetLastError();
}

// ---- tile tables ----------------------------------------------------------------------------------------------------
// Grouped: group g owns token rows [offsets[g], offsets[g+1]) and weight rows [g * Nn, (g + 1) * Nn) (pair: gate rows
// [g * 2I, g * 2I + I), up rows behind them, Nn = I output columns).  Tiles of a group: token blocks outermost.
__global__ void fp4_build_tiles_kernel(Fp4Tile* __restrict__ tiles, int* __restrict__ num_tiles, const int* __restrict__ offsets,
                                       int groups, int Nn, int pair, int bn, int max_tiles) {
    pdl_grid_sync();
    __shared__ int base[1025];
    const int g = threadIdx.x;
    const int mt = Nn / BM;                               // weight-row tiles per group
    const int rows_per_group = pair ? 2 * Nn : Nn;
    const int blks_per_group = rows_per_group / BM;
    int mine = 0;
    if (g < groups) mine = ((offsets[g + 1] - offsets[g] + bn - 1) / bn) * mt;
    base[g + 1] = mine;
    if (g == 0) base[0] = 0;
    __syncthreads();
    if (g == 0) for (int i = 1; i <= groups; ++i) base[i] += base[i - 1];
    __syncthreads();
    if (g < groups) {
        int at = base[g];
        const int r0 = offsets[g], r1 = offsets[g + 1];
        for (int b = r0; b < r1; b += bn)
            for (int m = 0; m < mt; ++m, ++at)
                if (at < max_tiles) {
                    Fp4Tile t;
                    t.a_row0 = g * rows_per_group + m * BM;
                    t.a_row1 = pair ? g * rows_per_group + Nn + m * BM : -1;
                    t.sfa_blk0 = g * blks_per_group + m;
                    t.sfa_blk1 = pair ? g * blks_per_group + mt + m : -1;
                    t.b_row0 = b;
                    t.b_valid = min(bn, r1 - b);
                    t.out_n0 = m * BM;
                    t.group = g;
                    tiles[at] = t;
                }
    }
    if (g == 0) *num_tiles = min(base[groups], max_tiles);
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
// One block per output row: out row m = NVFP4 of x[src[m]] (or x[m]); per-row global scale g = amax / (6 * 448), block
// scale = e4m3(amax_16 / (6 g)), code = e2m1(x / (scale * g)).  With `terms` > 1 row m + j * rows holds the j-th residual
// (what the first j terms left over), quantised the same way.  Rows whose source is outside x are zero.
__global__ void __launch_bounds__(256) nvfp4_quantize_rows_kernel(uint8_t* __restrict__ q, uint8_t* __restrict__ sf, float* __restrict__ g,
                                                                   const bf16* __restrict__ x, const int* __restrict__ src, int rows,
                                                                   int x_rows, int K, int ldx, int terms) {
    pdl_grid_sync();
    extern __shared__ float xrow[];                 // [K] what is left to represent
    __shared__ float scratch[33];
    const int m = blockIdx.x;
    const size_t total_rows = (size_t)rows * terms;
    const int sr = src ? src[m] : m;
    const bool valid = sr >= 0 && sr < x_rows;
    for (int i = threadIdx.x; i < K; i += blockDim.x) xrow[i] = valid ? __bfloat162float(x[(size_t)sr * ldx + i]) : 0.f;
    __syncthreads();
    for (int term = 0; term < terms; ++term) {
        const size_t orow = (size_t)m + (size_t)term * rows;
        float amax = 0.f;
        for (int i = threadIdx.x; i < K; i += blockDim.x) amax = fmaxf(amax, fabsf(xrow[i]));
        amax = block_max(amax, scratch);
        const float gs = amax > 0.f ? amax / (6.f * 448.f) : 1.f;
        if (threadIdx.x == 0) g[orow] = gs;
        const float inv_g = 1.f / gs;
        // one thread per block of 16 values
        for (int b = threadIdx.x; b < K / 16; b += blockDim.x) {
            float* v = xrow + b * 16;
            float bm = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) bm = fmaxf(bm, fabsf(v[i]));
            const uint8_t sc8 = float_to_e4m3(bm * inv_g * (1.f / 6.f));
            const float sc = e4m3_to_float(sc8);
            const float dq = sc * gs;                                   // value of code 1.0
            const float inv = dq > 0.f ? 1.f / dq : 0.f;
            uint32_t packed[2] = {0u, 0u};
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
                uint32_t two;
                // d = {e2m1(b), e2m1(a)}: the first source lands in the high nibble
                asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u32.u8 %0, t; }" : "=r"(two) : "f"(v[i + 1] * inv), "f"(v[i] * inv));
                packed[i / 8] |= two << (4 * (i % 8));
                if (terms > 1) {
                    // what this term represents, taken off the remainder
                    const int c0 = two & 0xF, c1 = (two >> 4) & 0xF;
                    const float tab[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
                    const float d0 = (c0 & 8 ? -tab[c0 & 7] : tab[c0 & 7]) * dq, d1 = (c1 & 8 ? -tab[c1 & 7] : tab[c1 & 7]) * dq;
                    v[i] -= d0; v[i + 1] -= d1;
                }
            }
            *reinterpret_cast<uint2*>(q + orow * (K / 2) + (size_t)b * 8) = make_uint2(packed[0], packed[1]);
            sf[((size_t)(b / 4) * total_rows + orow) * 16 + (b % 4)] = sc8;
        }
        __syncthreads();
    }
}

template <int PAIR>
int dispatch_bn(int bn, const void* W, int w_rows, const void* X, int x_rows, const void* sfb, const Fp4Params& p, int max_tiles, cudaStream_t s) {
    switch (bn) {
        case 32: return launch_fp4<32, PAIR>(W, w_rows, X, x_rows, sfb, p, max_tiles, s);
        case 64: return launch_fp4<64, PAIR>(W, w_rows, X, x_rows, sfb, p, max_tiles, s);
        case 128: return launch_fp4<128, PAIR>(W, w_rows, X, x_rows, sfb, p, max_tiles, s);
        default: return -1;
    }
}

}  // namespace

// Bytes per tile-table entry (the caller allocates max_tiles of them).
SL_API int sl_fp4_tile_bytes() { return (int)sizeof(Fp4Tile); }

// Tile table of a grouped product: `offsets` int32 [groups + 1] on the device, Nn output columns per group
// (a multiple of 128), `pair` = gate/up weight stacks [groups][2 Nn][K/2] with the SiLU * mul epilogue.
SL_API int sl_fp4_build_tiles(void* tiles, void* num_tiles, const void* offsets, int groups, int Nn, int pair, int bn, int max_tiles,
                              cudaStream_t s) {
    if (groups <= 0 || groups > 1024 || Nn % BM != 0 || (bn != 32 && bn != 64 && bn != 128)) return -1;
    sl_launch(fp4_build_tiles_kernel, 1, 1024, 0, s, (Fp4Tile*)tiles, (int*)num_tiles, (const int*)offsets, groups, Nn, pair, bn, max_tiles);
    return (int)cudaGetLastError();
}

// Grouped (or, with one group, plain) NVFP4 x NVFP4 product over a tile table.
//   W [w_rows, K/2] packed weights, sfa their scale tiles, gA [groups] (pair: [groups][2]) fp32
//   X [x_rows, K/2] packed activation rows, sfb [K/64][x_rows][16] their scales (see the file header), gB [x_rows] fp32
//   out [x_rows, ldo] bf16 (out_kind 0) or fp32 (1); pair: out = silu(gate) * up, Nn = I columns
// K % 256 == 0.  `err` is set to a non-zero site code when a bounded wait expired.
SL_API int sl_gemm_fp4_tcgen05(const void* W, const void* sfa, const void* gA, int w_rows, const void* X, const void* sfb, const void* gB,
                               int x_rows, void* out, int ldo, int out_kind, int K, int pair, int bn, const void* tiles,
                               const void* num_tiles, int max_tiles, void* err, cudaStream_t s) {
    if (w_rows <= 0 || x_rows <= 0 || max_tiles <= 0) return 0;
    if (K % 256 != 0 || K <= 0) return -1;
    Fp4Params p{};
    p.sfa = (const uint8_t*)sfa; p.gA = (const float*)gA; p.gB = (const float*)gB; p.out = out; p.K = K; p.ldo = ldo;
    p.out_kind = out_kind; p.tiles = (const Fp4Tile*)tiles; p.num_tiles = (const int*)num_tiles;
    p.err = (int*)err;
    return pair ? dispatch_bn<1>(bn, W, w_rows, X, x_rows, sfb, p, max_tiles, s) : dispatch_bn<0>(bn, W, w_rows, X, x_rows, sfb, p, max_tiles, s);
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

// bf16 rows -> NVFP4 rows (+ residual terms).  q [rows * terms, K/2], sf [K/64][rows * terms][16] (four scales, then
// padding), g [rows * terms]; `src` (int32 [rows], may be null) gathers: output row m quantises x[src[m]].
// K % 64 == 0, K <= 16384.
SL_API int sl_nvfp4_quantize_rows(void* q, void* sf, void* g, const void* x, const void* src, int rows, int x_rows, int K, int ldx,
                                  int terms, cudaStream_t s) {
    if (rows <= 0) return 0;
    if (K % 64 != 0 || K > 16384 || terms < 1 || terms > 4) return -1;
    const size_t smem = (size_t)K * sizeof(float);
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(nvfp4_quantize_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 16384 * (int)sizeof(float));
        attr_set = true;
    }
    sl_launch(nvfp4_quantize_rows_kernel, rows, 256, smem, s, (uint8_t*)q, (uint8_t*)sf, (float*)g, (const bf16*)x, (const int*)src, rows,
              x_rows, K, ldx, terms);
    return (int)cudaGetLastError();
}
