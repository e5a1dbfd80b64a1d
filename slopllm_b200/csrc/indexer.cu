// DSA lightning indexer: FP8 scoring of a query token's 32x128 index heads against this
// rank's paged FP8 key rows, and exact top-k selection with ascending-index output.
//
// score[j] = kscale[j] * sum_h w_eff[h] * relu(q8[h] . k8[j])
//
// Reference: `csrc/glm_indexer.cu:1375-1510` (fp8 mma scoring), `:490-870` (radix top-k,
// stable gather, sort by index).  Here scoring runs on the FP8 tensor path with fp32
// scores, the select is a 4x8-bit radix descent over order-preserving keys, and the gather
// emits ascending positions directly (no separate sort).
#include "indexer.cuh"

__device__ __forceinline__ void mma_e4m3_m16n8k32(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// grid (key tiles of 8 warps x 8 keys x ITER, T); Hi == 32, D == 128.
// The 128-byte key row is consumed with a fixed permutation of the reduction index that is
// applied to Q as well, so every lane issues two 16-byte loads per key row quarter.
template <int HI, int D>
__global__ void __launch_bounds__(256) indexer_score_kernel(IndexerScoreParams p, int keys_per_block) {
    pdl_grid_sync();
    static_assert(HI % 16 == 0 && D % 32 == 0, "index heads / dim");
    constexpr int MT = HI / 16;          // m tiles (16 heads each)
    constexpr int KS = D / 32;           // k steps of 32
    const int t = blockIdx.y;
    const int pos = p.positions[t];
    if (pos + 1 <= p.top_k) return;      // everything visible is selected: no scores needed
    const int n_local = local_visible(pos, p.cp_world, p.cp_rank);
    const int k_begin = blockIdx.x * keys_per_block;
    if (k_begin >= n_local) return;
    const int k_end = min(n_local, k_begin + keys_per_block);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, c = lane & 3;
    constexpr int RB = D + 4;

    // A fragments: logical k (s, half, c, i) <-> dim c*(D/4) + s*8 + half*4 + i
    uint32_t a[MT][KS][4];
    float w[MT][2];
    const uint8_t* q = p.q8 + (size_t)t * HI * D;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
#pragma unroll
        for (int s = 0; s < KS; ++s) {
            const int d0 = c * (D / 4) + s * 8;
            a[m][s][0] = *reinterpret_cast<const uint32_t*>(q + (size_t)(m * 16 + g) * D + d0);
            a[m][s][1] = *reinterpret_cast<const uint32_t*>(q + (size_t)(m * 16 + g + 8) * D + d0);
            a[m][s][2] = *reinterpret_cast<const uint32_t*>(q + (size_t)(m * 16 + g) * D + d0 + 4);
            a[m][s][3] = *reinterpret_cast<const uint32_t*>(q + (size_t)(m * 16 + g + 8) * D + d0 + 4);
        }
        w[m][0] = p.w_eff[(size_t)t * HI + m * 16 + g];
        w[m][1] = p.w_eff[(size_t)t * HI + m * 16 + g + 8];
    }
    const int* pt = p.page_table + (size_t)p.batch_idx[t] * p.pt_stride;
    for (int j0 = k_begin + warp * 8; j0 < k_end; j0 += 64) {
        // lane's key for the B fragment: j0 + g ; 8 consecutive keys never straddle a page
        const int j = j0 + g;
        bool ok = j < k_end;
        const int pidx = j0 / p.page_size;
        if (!guard_ok(p.guard, 21, pidx, p.pt_stride)) continue;            // warp-uniform
        const size_t slot = (size_t)pt[pidx] * p.page_size + (j0 % p.page_size) + g;
        if (ok && p.num_slots != 0 && !guard_ok(p.guard, 22, (long long)slot, p.num_slots)) ok = false;
        const uint8_t* row = p.idx_cache + slot * RB;
        uint32_t b[KS][2];
        // row stride D+4 keeps 4-byte alignment only: read the lane's 32 bytes as 8 words
#pragma unroll
        for (int s = 0; s < KS; ++s) {
            b[s][0] = ok ? *reinterpret_cast<const uint32_t*>(row + c * (D / 4) + s * 8) : 0u;
            b[s][1] = ok ? *reinterpret_cast<const uint32_t*>(row + c * (D / 4) + s * 8 + 4) : 0u;
        }
        float part[2] = {0.f, 0.f};       // keys 2c, 2c+1 of this group of 8
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < KS; ++s) mma_e4m3_m16n8k32(d, a[m][s], b[s]);
            part[0] += w[m][0] * fmaxf(d[0], 0.f) + w[m][1] * fmaxf(d[2], 0.f);
            part[1] += w[m][0] * fmaxf(d[1], 0.f) + w[m][1] * fmaxf(d[3], 0.f);
        }
        // reduce over the 8 row groups g (lanes with equal c)
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            part[0] += __shfl_xor_sync(0xffffffffu, part[0], o);
            part[1] += __shfl_xor_sync(0xffffffffu, part[1], o);
        }
        if (g == 0) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int jj = j0 + 2 * c + i;
                if (jj < k_end) {
                    const size_t sl = (size_t)pt[j0 / p.page_size] * p.page_size + (j0 % p.page_size) + 2 * c + i;
                    if (p.num_slots != 0 && !guard_ok(p.guard, 23, (long long)sl, p.num_slots)) continue;
                    const float ks = *reinterpret_cast<const float*>(p.idx_cache + sl * RB + D);
                    p.scores[(size_t)t * p.ld_scores + jj] = part[i] * ks;
                }
            }
        }
    }
}

// Prefill form: one CTA scores 8 consecutive query tokens (one per warp) against the same key tiles.  When the 8 tokens
// belong to one sequence (a prefill chunk) a 64-key page (64 x 132 contiguous bytes) is copied into shared memory once
// with 16-byte loads and all 8 warps take their B fragments from there, so each key row crosses L2 once per 8 tokens
// instead of once per token with 4-byte loads; the next page is held in registers while the current one is multiplied.
// Groups that mix sequences fall back to per-warp loads from the cache.  Same fragment layout and accumulation order as
// the per-token kernel: the scores are bit-identical.  page_size == 64, keys_per_block a multiple of 64.
bool g_indexer_tiled = true;

template <int HI, int D>
__global__ void __launch_bounds__(256) indexer_score_tile_kernel(IndexerScoreParams p, int T, int keys_per_block) {
    pdl_grid_sync();
    constexpr int MT = HI / 16, KS = D / 32, RB = D + 4, PAGE = 64;
    constexpr int PAGE_BYTES = PAGE * RB;                 // 8448 = 528 x 16
    constexpr int PIECES = PAGE_BYTES / 16, LD = (PIECES + 255) / 256;
    static_assert(PAGE_BYTES % 16 == 0, "a page is a whole number of 16-byte pieces");
    __shared__ __align__(16) uint8_t tile[PAGE_BYTES];
    __shared__ int s_bidx[8], s_nloc[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, c = lane & 3;
    const int t = blockIdx.y * 8 + warp;
    const bool live = t < T;
    const int pos = live ? p.positions[t] : -1;
    // tokens whose visible keys are all selected need no scores
    const int n_local = (live && pos + 1 > p.top_k) ? local_visible(pos, p.cp_world, p.cp_rank) : 0;
    if (lane == 0) { s_bidx[warp] = live ? p.batch_idx[t] : -1; s_nloc[warp] = n_local; }
    __syncthreads();
    int n_max = 0;
    bool same = true;
    int b0 = -1;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        n_max = max(n_max, s_nloc[i]);
        if (s_nloc[i] > 0) { if (b0 < 0) b0 = s_bidx[i]; else same = same && (s_bidx[i] == b0); }
    }
    const int k_begin = blockIdx.x * keys_per_block;
    if (k_begin >= n_max) return;                          // CTA-uniform
    const int k_end_cta = min(n_max, k_begin + keys_per_block);
    const int k_end = min(n_local, k_end_cta);             // this warp's bound (may be below k_begin)

    uint32_t a[MT][KS][4];
    float w[MT][2];
    if (n_local > 0) {
        const uint8_t* q = p.q8 + (size_t)t * HI * D;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
#pragma unroll
            for (int s = 0; s < KS; ++s) {
                const int d0 = c * (D / 4) + s * 8;
                a[m][s][0] = *reinterpret_cast<const uint32_t*>(q + (size_t)(m * 16 + g) * D + d0);
                a[m][s][1] = *reinterpret_cast<const uint32_t*>(q + (size_t)(m * 16 + g + 8) * D + d0);
                a[m][s][2] = *reinterpret_cast<const uint32_t*>(q + (size_t)(m * 16 + g) * D + d0 + 4);
                a[m][s][3] = *reinterpret_cast<const uint32_t*>(q + (size_t)(m * 16 + g + 8) * D + d0 + 4);
            }
            w[m][0] = p.w_eff[(size_t)t * HI + m * 16 + g];
            w[m][1] = p.w_eff[(size_t)t * HI + m * 16 + g + 8];
        }
    } else {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
#pragma unroll
            for (int s = 0; s < KS; ++s) a[m][s][0] = a[m][s][1] = a[m][s][2] = a[m][s][3] = 0u;
            w[m][0] = w[m][1] = 0.f;
        }
    }
    // scores of the 8 keys [j0, j0 + 8) from B fragments at `rows` (row stride RB); keys at or beyond k_end are not written
    auto score8 = [&](const uint8_t* rows, int j0) {
        const uint8_t* row = rows + g * RB;
        uint32_t b[KS][2];
#pragma unroll
        for (int s = 0; s < KS; ++s) {
            b[s][0] = *reinterpret_cast<const uint32_t*>(row + c * (D / 4) + s * 8);
            b[s][1] = *reinterpret_cast<const uint32_t*>(row + c * (D / 4) + s * 8 + 4);
        }
        float part[2] = {0.f, 0.f};
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < KS; ++s) mma_e4m3_m16n8k32(d, a[m][s], b[s]);
            part[0] += w[m][0] * fmaxf(d[0], 0.f) + w[m][1] * fmaxf(d[2], 0.f);
            part[1] += w[m][0] * fmaxf(d[1], 0.f) + w[m][1] * fmaxf(d[3], 0.f);
        }
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            part[0] += __shfl_xor_sync(0xffffffffu, part[0], o);
            part[1] += __shfl_xor_sync(0xffffffffu, part[1], o);
        }
        if (g == 0) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int jj = j0 + 2 * c + i;
                if (jj < k_end) p.scores[(size_t)t * p.ld_scores + jj] = part[i] * *reinterpret_cast<const float*>(rows + (2 * c + i) * RB + D);
            }
        }
    };

    if (same) {
        const int* pt = p.page_table + (size_t)b0 * p.pt_stride;
        uint4 nxt[LD];
        auto fetch = [&](int j0) {                         // the page of local keys [j0, j0 + 64) into registers
            const int pidx = j0 / PAGE;
            bool ok = guard_ok(p.guard, 21, pidx, p.pt_stride);
            long long base = 0;
            if (ok) {
                base = (long long)pt[pidx] * PAGE;
                if (p.num_slots != 0 && !guard_ok(p.guard, 22, base + PAGE - 1, p.num_slots)) ok = false;
            }
            const uint8_t* src = p.idx_cache + (size_t)base * RB;
#pragma unroll
            for (int i = 0; i < LD; ++i) {
                const int piece = threadIdx.x + i * 256;
                nxt[i] = (ok && piece < PIECES) ? ldg_nc_16(src + piece * 16) : make_uint4(0u, 0u, 0u, 0u);
            }
        };
        fetch(k_begin);
        for (int j0 = k_begin; j0 < k_end_cta; j0 += PAGE) {
            __syncthreads();                               // every warp is done with the previous page
#pragma unroll
            for (int i = 0; i < LD; ++i) {
                const int piece = threadIdx.x + i * 256;
                if (piece < PIECES) *reinterpret_cast<uint4*>(tile + piece * 16) = nxt[i];
            }
            __syncthreads();
            if (j0 + PAGE < k_end_cta) fetch(j0 + PAGE);
            if (j0 < k_end) {                              // warp-uniform
#pragma unroll 2
                for (int nt = 0; nt < PAGE / 8; ++nt)
                    if (j0 + nt * 8 < k_end) score8(tile + nt * 8 * RB, j0 + nt * 8);
            }
        }
    } else if (n_local > 0) {
        const int* pt = p.page_table + (size_t)p.batch_idx[t] * p.pt_stride;
        for (int j0 = k_begin; j0 < k_end; j0 += 8) {
            const int pidx = j0 / p.page_size;
            if (!guard_ok(p.guard, 21, pidx, p.pt_stride)) continue;
            const size_t slot = (size_t)pt[pidx] * p.page_size + (j0 % p.page_size);
            if (p.num_slots != 0 && !guard_ok(p.guard, 22, (long long)slot + 7, p.num_slots)) continue;
            score8(p.idx_cache + slot * RB, j0);
        }
    }
}

// Generic CUDA-core scorer for other head counts / dims (small test models).
__global__ void indexer_score_generic_kernel(IndexerScoreParams p, int keys_per_block) {
    pdl_grid_sync();
    extern __shared__ float qs[];          // [Hi*D] + [Hi]
    const int t = blockIdx.y;
    const int pos = p.positions[t];
    if (pos + 1 <= p.top_k) return;
    const int n_local = local_visible(pos, p.cp_world, p.cp_rank);
    const int k_begin = blockIdx.x * keys_per_block;
    if (k_begin >= n_local) return;
    const int k_end = min(n_local, k_begin + keys_per_block);
    float* ws = qs + p.Hi * p.D;
    for (int i = threadIdx.x; i < p.Hi * p.D; i += blockDim.x) qs[i] = e4m3_to_float(p.q8[(size_t)t * p.Hi * p.D + i]);
    for (int i = threadIdx.x; i < p.Hi; i += blockDim.x) ws[i] = p.w_eff[(size_t)t * p.Hi + i];
    __syncthreads();
    const int* pt = p.page_table + (size_t)p.batch_idx[t] * p.pt_stride;
    const int RB = p.D + 4;
    for (int j = k_begin + threadIdx.x; j < k_end; j += blockDim.x) {
        if (!guard_ok(p.guard, 24, j / p.page_size, p.pt_stride)) continue;
        const size_t slot = (size_t)pt[j / p.page_size] * p.page_size + (j % p.page_size);
        if (p.num_slots != 0 && !guard_ok(p.guard, 25, (long long)slot, p.num_slots)) continue;
        const uint8_t* row = p.idx_cache + slot * RB;
        float tot = 0.f;
        for (int h = 0; h < p.Hi; ++h) {
            float dot = 0.f;
            for (int d = 0; d < p.D; ++d) dot += qs[h * p.D + d] * e4m3_to_float(row[d]);
            tot += ws[h] * fmaxf(dot, 0.f);
        }
        p.scores[(size_t)t * p.ld_scores + j] = tot * *reinterpret_cast<const float*>(row + p.D);
    }
}

SL_API int sl_indexer_scores(const IndexerScoreParams* p, int T, int max_local, cudaStream_t s) {
    if (T == 0 || max_local <= 0) return 0;
    // tile the keys so that the grid has a few waves of blocks
    int kpb = 512;
    while (kpb > 64 && (long)((max_local + kpb - 1) / kpb) * T < 296) kpb >>= 1;
    dim3 grid((max_local + kpb - 1) / kpb, T);
    {
        const int rc = indexer_scores_tcgen05(p, T, max_local, s);
        if (rc != -2) return rc;
    }
    if (p->Hi == 32 && p->D == 128 && p->page_size == 64 && T > 32 && g_indexer_tiled) {
        // prefill: 8 tokens per CTA share the key pages
        const int groups = (T + 7) / 8;
        int kt = 2048;
        while (kt > 64 && (long)((max_local + kt - 1) / kt) * groups < 296) kt >>= 1;
        sl_launch(indexer_score_tile_kernel<32, 128>, dim3((max_local + kt - 1) / kt, groups), 256, 0, s, *p, T, kt);
    } else if (p->Hi == 32 && p->D == 128) {
        sl_launch(indexer_score_kernel<32, 128>, grid, 256, 0, s, *p, kpb);
    } else {
        const size_t smem = (size_t)(p->Hi * p->D + p->Hi) * sizeof(float);
        if (smem > 48 * 1024) return -1;
        sl_launch(indexer_score_generic_kernel, grid, 256, smem, s, *p, kpb);
    }
    return SL_LAUNCH_CHECK();
}

// 0 keeps the per-token kernel for every shape (comparison runs); default 1.
SL_API void sl_indexer_set_tiled(int on) { g_indexer_tiled = on != 0; }

// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t order_key(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct TopkSelectParams {
    const float* scores; int ld_scores;
    const int* positions;
    int top_k, cp_world, cp_rank;
    int* out_pos;             // [T, top_k] global positions ascending, -1 padded
    float* out_score;         // [T, top_k] (0 where unused)
    // optional fused slot lookup (cp_world == 1 only; null to skip): physical cache slots of the
    // selected keys in the same order, -1 padded, and the number selected per token
    int* slots; int* lengths;
    const int* page_table; const int* batch_idx;
    int pt_stride, page_size;
    // plain mode (n_fixed > 0): every row has exactly n_fixed candidates and the output is the candidate index
    // (used to merge the ranks' candidate lists under context parallelism); `positions` is not read
    int n_fixed;
};

// Radix-descent helper: given hist[256] of the current digit among the candidates, find the bin
// that contains the `rem`-th largest and update (prefix, remaining).  Threads 0..255 take part;
// bins are scanned from the top with warp shuffles.  Must be called by the whole block.
__device__ __forceinline__ void radix_pick_bin(const uint32_t* hist, uint32_t* wtot, uint32_t* s_prefix, uint32_t* s_remaining,
                                               uint32_t prefix, int shift) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t rem = *s_remaining;             // read before anyone may update it (barrier below)
    uint32_t v = 0, incl = 0;
    if (tid < 256) {
        v = hist[255 - tid];                       // reversed: prefix sums run from the top bin down
        incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
        }
        if (lane == 31) wtot[warp] = incl;
    }
    __syncthreads();
    if (tid < 256) {
        uint32_t base = 0;
        for (int w = 0; w < warp; ++w) base += wtot[w];
        incl += base;
        const uint32_t above = incl - v;
        if (above < rem && incl >= rem) {          // exactly one bin satisfies this
            *s_prefix = prefix | ((uint32_t)(255 - tid) << shift);
            *s_remaining = rem - above;
        }
    }
    __syncthreads();
}

// One block per query token.  If the query sees at most top_k keys in total, all local keys are emitted.
// Otherwise: radix descent for the k'-th largest key (k' = min(top_k, n_local)) over four 8-bit digits, then an
// in-order gather of keys above the threshold plus the first ties.
//   * digit histograms are private to a warp (32 x 256 counters in shared memory) and lanes that hit the same bin
//     are merged with a warp match first, so the scan needs no atomics and does not serialise on the few bins that
//     similar scores share;
//   * the gather gives every warp one contiguous segment of the row: a counting walk, one scan over the 32 warps'
//     totals, and an emitting walk with warp-local running offsets, instead of block-wide barriers per 1024 keys.
// The row (at most a few hundred KB) stays in L1 / L2 between the six walks.
__global__ void __launch_bounds__(1024) topk_select_kernel(TopkSelectParams p) {
    pdl_grid_sync();
    __shared__ uint32_t whist[32][256];
    __shared__ uint32_t hist[256];
    __shared__ uint32_t wtot[8];
    __shared__ uint32_t s_prefix, s_remaining;
    __shared__ int wgt[32], weq[32];
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pos = p.n_fixed > 0 ? p.n_fixed - 1 : p.positions[t];
    const int n = p.n_fixed > 0 ? p.n_fixed : local_visible(pos, p.cp_world, p.cp_rank);
    int* opos = p.out_pos + (size_t)t * p.top_k;
    float* osc = p.out_score + (size_t)t * p.top_k;
    int* oslot = p.slots != nullptr ? p.slots + (size_t)t * p.top_k : nullptr;
    const int* pt = p.slots != nullptr ? p.page_table + (size_t)p.batch_idx[t] * p.pt_stride : nullptr;
    if (pos + 1 <= p.top_k) {
        for (int i = tid; i < p.top_k; i += blockDim.x) {
            opos[i] = i < n ? i * p.cp_world + p.cp_rank : -1;
            osc[i] = 0.f;
            if (oslot != nullptr) oslot[i] = i < n ? pt[i / p.page_size] * p.page_size + i % p.page_size : -1;
        }
        if (oslot != nullptr && tid == 0) p.lengths[t] = n;
        return;
    }
    const float* sc = p.scores + (size_t)t * p.ld_scores;
    const bool vec = (((uintptr_t)sc) & 15) == 0 && p.ld_scores % 4 == 0;      // whole groups of 4 stay inside the row
    const int kk = min(p.top_k, n);
    // warp w owns keys [lo, hi) in every walk (segments are whole groups of 128 keys)
    const int seg = ((n + 31) / 32 + 127) / 128 * 128;
    const int lo = min(n, warp * seg), hi = min(n, lo + seg);
    uint32_t mask = 0;
    int above24 = 0;                               // last digit's walk: keys of this lane whose upper 24 bits exceed the threshold's
    if (tid == 0) { s_prefix = 0; s_remaining = (uint32_t)kk; }
    uint32_t* mine = whist[warp];
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = tid; i < 32 * 256; i += 1024) (&whist[0][0])[i] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        auto visit = [&](bool live, float v) {
            const uint32_t key = order_key(v);
            const bool hit = live && (key & mask) == prefix;
            if (shift == 0 && live && (key & mask) > prefix) ++above24;
            const unsigned hm = __ballot_sync(0xffffffffu, hit);
            if (hm == 0) return;                   // warp-uniform: nothing of this group is still a candidate
            if (hit) {
                const uint32_t bin = (key >> shift) & 255u;
                const unsigned peers = __match_any_sync(hm, bin);
                if (lane == __ffs(peers) - 1) mine[bin] += __popc(peers);
            }
            __syncwarp();
        };
        // every lane of a warp makes the same number of trips (the visits vote)
        if (vec) {
            for (int b0 = lo; b0 < hi; b0 += 128) {
                const int i0 = b0 + lane * 4;
                const float4 v = i0 < hi ? *reinterpret_cast<const float4*>(sc + i0) : make_float4(0.f, 0.f, 0.f, 0.f);
                visit(i0 < hi, v.x); visit(i0 + 1 < hi, v.y); visit(i0 + 2 < hi, v.z); visit(i0 + 3 < hi, v.w);
            }
        } else {
            for (int b0 = lo; b0 < hi; b0 += 32) {
                const int i = b0 + lane;
                visit(i < hi, i < hi ? sc[i] : 0.f);
            }
        }
        __syncthreads();
        if (tid < 256) {
            uint32_t c = 0;
#pragma unroll 8
            for (int w = 0; w < 32; ++w) c += whist[w][tid];
            hist[tid] = c;
        }
        __syncthreads();
        radix_pick_bin(hist, wtot, &s_prefix, &s_remaining, prefix, shift);
        mask |= 0xffu << shift;
    }
    const uint32_t thr = s_prefix;
    const int need_eq = (int)s_remaining;      // how many keys equal to thr are taken (lowest index first)
    // this warp's keys above / at the threshold: those decided by the upper 24 bits, plus the last digit's private
    // histogram (it still holds exactly this warp's candidates by low byte)
    {
        const int tl = (int)(thr & 255u);
        int g = above24, e = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int bin = lane * 8 + i;
            const int c = (int)mine[bin];
            g += bin > tl ? c : 0;
            e += bin == tl ? c : 0;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            g += __shfl_xor_sync(0xffffffffu, g, o);
            e += __shfl_xor_sync(0xffffffffu, e, o);
        }
        if (lane == 0) { wgt[warp] = g; weq[warp] = e; }
    }
    __syncthreads();
    int base = 0, eq_used = 0;
    for (int w = 0; w < warp; ++w) {
        const int e = weq[w];
        base += wgt[w] + max(0, min(e, need_eq - eq_used));
        eq_used += e;
    }
    const unsigned lt = (1u << lane) - 1;
    for (int i0 = lo; i0 < hi; i0 += 32) {
        const int i = i0 + lane;
        const float v = i < hi ? sc[i] : 0.f;
        const uint32_t key = i < hi ? order_key(v) : 0u;
        const bool gt = i < hi && key > thr, eq = i < hi && key == thr;
        const unsigned meq = __ballot_sync(0xffffffffu, eq);
        const bool take = gt || (eq && eq_used + __popc(meq & lt) < need_eq);
        const unsigned mt = __ballot_sync(0xffffffffu, take);
        const int off = base + __popc(mt & lt);
        if (take && off < p.top_k) {
            opos[off] = i * p.cp_world + p.cp_rank;
            osc[off] = v;
            if (oslot != nullptr) oslot[off] = pt[i / p.page_size] * p.page_size + i % p.page_size;
        }
        base += __popc(mt);
        eq_used += __popc(meq);
    }
    // the last warp's running total is the number selected
    __shared__ int s_total;
    if (warp == 31 && lane == 0) s_total = base;
    __syncthreads();
    const int total = s_total;
    for (int i = total + tid; i < p.top_k; i += blockDim.x) {
        opos[i] = -1;
        osc[i] = 0.f;
        if (oslot != nullptr) oslot[i] = -1;
    }
    if (oslot != nullptr && tid == 0) p.lengths[t] = min(total, p.top_k);
}

SL_API int sl_topk_select(const TopkSelectParams* p, int T, cudaStream_t s) {
    if (T == 0) return 0;
    if (p->slots != nullptr && p->cp_world != 1) return -1;
    sl_launch(topk_select_kernel, T, 1024, 0, s, *p);
    return SL_LAUNCH_CHECK();
}
