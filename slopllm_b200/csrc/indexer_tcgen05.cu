// DSA lightning indexer, prefill form, on the 5th-generation tensor cores.
//
//   score[t, j] = kscale[j] * sum_h w_eff[t, h] * relu(q8[t, h, :] . k8[j, :])      32 heads, 128 dims, e4m3
//
// One CTA owns a block of up to 32 consecutive query tokens of one sequence and a range of 128-key tiles of that
// sequence's paged key rows.  The product is issued with the KEYS as the 128-row operand and (token, head) pairs as
// the 256 columns (8 tokens x 32 heads per `tcgen05.mma.kind::f8f6f4`, K = 128 in four instructions), so the
// accumulator of one key lives in one TMEM lane: the epilogue thread of that lane folds relu, head weights and the key
// scale over its 32 columns per token without any cross-thread traffic and the 32 lanes of a warp store 32 consecutive
// keys of a score row.  Per key tile the block's four token groups reuse the same shared-memory key tile, so a key row
// crosses L2 once per 32 tokens.
//
// Data movement: the queries of the block (128 KB) arrive once by TMA (128-byte swizzle); key pages (64 rows of
// 132 bytes = 128 e4m3 + fp32 scale, contiguous) arrive by untiled bulk copies into a raw ring and four warps re-lay
// them as a swizzled K-major tile (the 132-byte row pitch is not a TMA pitch), keeping the scales aside.
// Warp roles: 0 producer, 1 MMA issue (+ TMEM allocation), 2-5 re-layout, 6-13 epilogue (two per TMEM lane quarter,
// four tokens of the group each).  Two 256-column accumulators: the epilogue of one token group overlaps the MMAs of
// the next.  Every wait is bounded; on expiry the error word is set and all roles unwind.
//
// Reference: `csrc/glm_indexer.cu:1375-1510` (fp8 `mma.sync` scoring of the same quantity).
#include "indexer.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int HI = 32, D = 128, RB = D + 4, PAGE = 64;
constexpr int PAGE_BYTES = PAGE * RB;              // 8448
constexpr int TILE_KEYS = 128;                     // one MMA's rows: two pages
constexpr int TOK_GROUP = 8;                       // tokens per MMA (x 32 heads = 256 columns)
constexpr int MAX_GROUPS = 4;                      // token groups per CTA
constexpr int BLOCK_TOKENS = TOK_GROUP * MAX_GROUPS;
constexpr int Q_GROUP_BYTES = TOK_GROUP * HI * D;  // 32768
constexpr int A_BYTES = TILE_KEYS * D;             // 16384
constexpr int RAW_STAGES = 2, A_BUFS = 2, SCALE_BUFS = 4;
constexpr int RAW_BYTES = 2 * PAGE_BYTES;          // 16896
constexpr int THREADS = 14 * 32;
constexpr int EPI_WARP0 = 6, EPI_WARPS = 8;

// packed pairs of fp32 in one 64-bit register and their fused multiply-add (two lanes per instruction)
__device__ __forceinline__ unsigned long long pack2(float a, float b) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ float lo2(unsigned long long v) { return __uint_as_float((uint32_t)v); }
__device__ __forceinline__ float hi2(unsigned long long v) { return __uint_as_float((uint32_t)(v >> 32)); }

struct Smem {
    static constexpr int Q = 0;
    static constexpr int A = Q + MAX_GROUPS * Q_GROUP_BYTES;                 // 131072
    static constexpr int RAW = A + A_BUFS * A_BYTES;                         // 163840
    static constexpr int KSCALE = RAW + RAW_STAGES * RAW_BYTES;              // 197632
    static constexpr int WEFF = KSCALE + SCALE_BUFS * TILE_KEYS * 4;         // + 2048
    static constexpr int NLOC = WEFF + BLOCK_TOKENS * HI * 4;                // + 4096
    static constexpr int BARS = NLOC + BLOCK_TOKENS * 4;
    static constexpr int TOTAL = BARS + 16 * 8 + 16;
};
constexpr int SMEM_BYTES = Smem::TOTAL + 1024;     // + alignment slack

__global__ void __launch_bounds__(THREADS, 1)
indexer_score_tc_kernel(const __grid_constant__ CUtensorMap tmQ, IndexerScoreParams p, int T, int splits, int* __restrict__ err) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem + Smem::Q;
    uint8_t* sA = smem + Smem::A;
    uint8_t* sRaw = smem + Smem::RAW;
    float* sKs = reinterpret_cast<float*>(smem + Smem::KSCALE);
    float* sW = reinterpret_cast<float*>(smem + Smem::WEFF);
    int* sNloc = reinterpret_cast<int*>(smem + Smem::NLOC);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::BARS);
    uint64_t* q_full = bars;                   // [1]
    uint64_t* raw_full = bars + 1;             // [RAW_STAGES] pages landed (producer's bulk copies)
    uint64_t* raw_empty = raw_full + RAW_STAGES;   // [RAW_STAGES] re-layout has read the raw pages
    uint64_t* a_full = raw_empty + RAW_STAGES; // [A_BUFS] swizzled key tile written
    uint64_t* a_empty = a_full + A_BUFS;       // [A_BUFS] the MMAs that read it have finished
    uint64_t* acc_full = a_empty + A_BUFS;     // [2]
    uint64_t* acc_empty = acc_full + 2;        // [2]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0 && lane == 0) {
        tc::tma_prefetch_desc(&tmQ);
        tc::mbar_init(q_full, 1);
        for (int s = 0; s < RAW_STAGES; ++s) { tc::mbar_init(&raw_full[s], 1); tc::mbar_init(&raw_empty[s], 4); }
        for (int b = 0; b < A_BUFS; ++b) { tc::mbar_init(&a_full[b], 4); tc::mbar_init(&a_empty[b], 1); }
        for (int b = 0; b < 2; ++b) { tc::mbar_init(&acc_full[b], 1); tc::mbar_init(&acc_empty[b], EPI_WARPS); }
        tc::mbar_fence_init();
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_holder, 512);
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    pdl_grid_sync();

    // ---- this CTA's work: token block, key tiles ----
    const int t0 = blockIdx.x * BLOCK_TOKENS;
    const int ntok = min(BLOCK_TOKENS, T - t0);
    const int ngroups = (ntok + TOK_GROUP - 1) / TOK_GROUP;
    // tokens whose visible keys are all selected need no scores (the selection takes them all)
    auto visible = [&](int t) {
        const int pos = p.positions[t];
        return pos + 1 > p.top_k ? local_visible(pos, p.cp_world, p.cp_rank) : 0;
    };
    int n_max = 0;
    for (int i = 0; i < ntok; ++i) n_max = max(n_max, visible(t0 + i));     // positions ascend, but do not rely on it
    const int tiles_total = (n_max + TILE_KEYS - 1) / TILE_KEYS;
    const int per = (tiles_total + splits - 1) / splits;
    const int tile_begin = min(tiles_total, (int)blockIdx.y * per), tile_end = min(tiles_total, tile_begin + per);
    const int ntiles = tile_end - tile_begin;
    const int* pt = p.page_table + (size_t)p.batch_idx[t0] * p.pt_stride;
    const int pages_valid = (n_max + PAGE - 1) / PAGE;

    if (ntiles > 0) {
        if (warp == 0) {
            if (lane == 0) {
                tc::mbar_expect_tx(q_full, (uint32_t)(ngroups * Q_GROUP_BYTES));
                for (int g = 0; g < ngroups; ++g) tc::tma_load_2d(sQ + g * Q_GROUP_BYTES, &tmQ, q_full, 0, (t0 + g * TOK_GROUP) * HI);
                bool ok = true;
                for (int i = 0; i < ntiles && ok; ++i) {
                    const int s = i % RAW_STAGES;
                    if (!tc::mbar_wait(&raw_empty[s], ((i / RAW_STAGES) & 1) ^ 1)) { atomicExch(err, 21); ok = false; break; }
                    const int page0 = (tile_begin + i) * 2;
                    uint32_t bytes = 0;
                    long long base[2] = {-1, -1};
                    for (int pg = 0; pg < 2; ++pg) {
                        const int pidx = page0 + pg;
                        if (pidx >= pages_valid || !guard_ok(p.guard, 24, pidx, p.pt_stride)) continue;
                        const long long b = (long long)pt[pidx] * PAGE;
                        if (p.num_slots != 0 && !guard_ok(p.guard, 25, b + PAGE - 1, p.num_slots)) continue;
                        if (b < 0) continue;
                        base[pg] = b;
                        bytes += PAGE_BYTES;
                    }
                    if (bytes == 0) { tc::mbar_arrive(&raw_full[s]); continue; }
                    tc::mbar_expect_tx(&raw_full[s], bytes);
                    for (int pg = 0; pg < 2; ++pg)
                        if (base[pg] >= 0)
                            tc::bulk_load_1d(sRaw + s * RAW_BYTES + pg * PAGE_BYTES, p.idx_cache + (size_t)base[pg] * RB, PAGE_BYTES, &raw_full[s]);
                }
            }
        } else if (warp == 1) {
            if (lane == 0) {
                constexpr uint32_t idesc = tc::idesc_f8(TILE_KEYS, TOK_GROUP * HI);
                bool ok = tc::mbar_wait(q_full, 0);
                if (!ok) atomicExch(err, 22);
                int at = 0;                    // accumulator uses so far
                for (int i = 0; i < ntiles && ok; ++i) {
                    const int b = i % A_BUFS;
                    if (!tc::mbar_wait(&a_full[b], (i / A_BUFS) & 1)) { atomicExch(err, 23); ok = false; break; }
                    tc::fence_after_sync();
                    const uint32_t a_addr = tc::smem_u32(sA + b * A_BYTES);
                    for (int g = 0; g < ngroups; ++g, ++at) {
                        const int k = at & 1;
                        if (!tc::mbar_wait(&acc_empty[k], ((at >> 1) & 1) ^ 1)) { atomicExch(err, 24); ok = false; break; }
                        tc::fence_after_sync();
                        const uint32_t q_addr = tc::smem_u32(sQ + g * Q_GROUP_BYTES);
#pragma unroll
                        for (int ks = 0; ks < D / 32; ++ks)
                            tc::mma_f8_ss(tmem_base + k * 256, tc::smem_desc_sw128(a_addr + ks * 32), tc::smem_desc_sw128(q_addr + ks * 32),
                                          idesc, ks > 0 ? 1u : 0u);
                        tc::mma_commit(&acc_full[k]);
                    }
                    if (ok) tc::mma_commit(&a_empty[b]);
                }
            }
        } else if (warp < EPI_WARP0) {
            // re-layout: thread r of 128 owns key row r of the tile
            const int r = (warp - 2) * 32 + lane;
            const int pg = r / PAGE, rr = r % PAGE;
            bool ok = true;
            for (int i = 0; i < ntiles && ok; ++i) {
                const int s = i % RAW_STAGES, b = i % A_BUFS;
                if (!tc::mbar_wait(&raw_full[s], (i / RAW_STAGES) & 1)) { if (lane == 0) atomicExch(err, 25); ok = false; break; }
                if (!tc::mbar_wait(&a_empty[b], ((i / A_BUFS) & 1) ^ 1)) { if (lane == 0) atomicExch(err, 26); ok = false; break; }
                const bool have = (tile_begin + i) * 2 + pg < pages_valid;    // pages the producer skipped for other reasons hold stale
                const uint32_t* src = reinterpret_cast<const uint32_t*>(sRaw + s * RAW_BYTES + pg * PAGE_BYTES + rr * RB);   // bytes; masked below
                uint8_t* dst = sA + b * A_BYTES + r * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    uint4 v = make_uint4(0u, 0u, 0u, 0u);
                    if (have) { v.x = src[4 * c]; v.y = src[4 * c + 1]; v.z = src[4 * c + 2]; v.w = src[4 * c + 3]; }
                    *reinterpret_cast<uint4*>(dst + ((c ^ (r & 7)) << 4)) = v;
                }
                sKs[(i % SCALE_BUFS) * TILE_KEYS + r] = have ? __uint_as_float(src[D / 4]) : 0.f;
                tc::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) { tc::mbar_arrive(&a_full[b]); tc::mbar_arrive(&raw_empty[s]); }
            }
        } else {
            // epilogue: lane quarter q, tokens [half * 4, half * 4 + 4) of each group
            const int e = warp - EPI_WARP0, q = warp & 3, half = e >> 2;
            for (int i = threadIdx.x - EPI_WARP0 * 32; i < BLOCK_TOKENS * HI; i += EPI_WARPS * 32) {
                const int tl = i / HI;
                sW[i] = tl < ntok ? p.w_eff[(size_t)(t0 + tl) * HI + (i % HI)] : 0.f;
            }
            for (int i = threadIdx.x - EPI_WARP0 * 32; i < BLOCK_TOKENS; i += EPI_WARPS * 32) sNloc[i] = i < ntok ? visible(t0 + i) : 0;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            int at = 0;
            bool ok = true;
            for (int i = 0; i < ntiles && ok; ++i) {
                const int j = (tile_begin + i) * TILE_KEYS + q * 32 + lane;       // this thread's local key
                const float* ksb = sKs + (i % SCALE_BUFS) * TILE_KEYS;
                for (int g = 0; g < ngroups; ++g, ++at) {
                    const int k = at & 1;
                    if (!tc::mbar_wait(&acc_full[k], (at >> 1) & 1)) { if (lane == 0) atomicExch(err, 27); ok = false; break; }
                    tc::fence_after_sync();
                    const float ks = ksb[q * 32 + lane];      // written before a_full, which precedes acc_full
                    const uint32_t t_acc = tmem_base + ((uint32_t)(q * 32) << 16) + k * 256 + half * 128;
#pragma unroll
                    for (int pair = 0; pair < 2; ++pair) {
                        uint32_t r0[32], r1[32];
                        tc::tmem_ld_32x32(t_acc + (pair * 2) * 32, r0);
                        tc::tmem_ld_32x32(t_acc + (pair * 2 + 1) * 32, r1);
                        tc::tmem_ld_wait();
                        const int tl0 = g * TOK_GROUP + half * 4 + pair * 2;
                        const float4* w0 = reinterpret_cast<const float4*>(sW + tl0 * HI);
                        const float4* w1 = reinterpret_cast<const float4*>(sW + (tl0 + 1) * HI);
                        // two heads per packed FMA (fma.rn.f32x2): even heads accumulate in the low half, odd heads in the high
                        unsigned long long p0 = 0ull, p1 = 0ull;
#pragma unroll
                        for (int h4 = 0; h4 < HI / 4; ++h4) {
                            const float4 u = w0[h4], v = w1[h4];
                            p0 = fma2(pack2(u.x, u.y), pack2(fmaxf(__uint_as_float(r0[4 * h4]), 0.f), fmaxf(__uint_as_float(r0[4 * h4 + 1]), 0.f)), p0);
                            p0 = fma2(pack2(u.z, u.w), pack2(fmaxf(__uint_as_float(r0[4 * h4 + 2]), 0.f), fmaxf(__uint_as_float(r0[4 * h4 + 3]), 0.f)), p0);
                            p1 = fma2(pack2(v.x, v.y), pack2(fmaxf(__uint_as_float(r1[4 * h4]), 0.f), fmaxf(__uint_as_float(r1[4 * h4 + 1]), 0.f)), p1);
                            p1 = fma2(pack2(v.z, v.w), pack2(fmaxf(__uint_as_float(r1[4 * h4 + 2]), 0.f), fmaxf(__uint_as_float(r1[4 * h4 + 3]), 0.f)), p1);
                        }
                        const float a0 = lo2(p0) + hi2(p0), a1 = lo2(p1) + hi2(p1);
                        if (j < sNloc[tl0]) p.scores[(size_t)(t0 + tl0) * p.ld_scores + j] = a0 * ks;
                        if (j < sNloc[tl0 + 1]) p.scores[(size_t)(t0 + tl0 + 1) * p.ld_scores + j] = a1 * ks;
                    }
                    tc::fence_before_sync();
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(&acc_empty[k]);
                }
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace

bool g_indexer_tcgen05 = true;

int indexer_scores_tcgen05(const IndexerScoreParams* p, int T, int max_local, cudaStream_t s) {
    if (!g_indexer_tcgen05 || p->Hi != HI || p->D != D || p->page_size != PAGE || T <= 32 || p->err == nullptr || !p->one_sequence)
        return -2;
    if (((uintptr_t)p->q8 & 15) != 0 || ((uintptr_t)p->idx_cache & 15) != 0) return -2;
    CUtensorMap tmQ;
    if (make_tmap_2d(&tmQ, p->q8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)T * HI, D, D, TOK_GROUP * HI, D) != 0) return -2;
    const int blocks = (T + BLOCK_TOKENS - 1) / BLOCK_TOKENS;
    const int tiles = (max_local + TILE_KEYS - 1) / TILE_KEYS;
    // key splits: about four CTAs per SM in total, at least four tiles per CTA
    int splits = (4 * 148 + blocks - 1) / blocks;
    splits = max(1, min(splits, (tiles + 3) / 4));
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(indexer_score_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        attr_done = true;
    }
    sl_launch(indexer_score_tc_kernel, dim3(blocks, splits), THREADS, SMEM_BYTES, s, tmQ, *p, T, splits, p->err);
    return SL_LAUNCH_CHECK();
}

// 0 keeps the mma.sync kernels for every shape (comparison runs); default 1.
SL_API void sl_indexer_set_tcgen05(int on) { g_indexer_tcgen05 = on != 0; }
