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
#include "route.cuh"
#include "w4_frag.cuh"

namespace {

// ---- activation staging --------------------------------------------------------------------------
// x[T, K] bf16 -> f16 in fragment order in global scratch: 16-byte unit(token, group, j, c) holds
// x[token][group*128 + c*32 + j*8 .. +7] at unit index (token*G + group)*16 + j*4 + c, G = K/128.
// Rows T..tpad-1 are zero.
__device__ __forceinline__ void permute_x_unit(uint4* __restrict__ xp, const bf16* __restrict__ x, int i, int T, int K, int ldx) {
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

__global__ void permute_x_kernel(uint4* __restrict__ xp, const bf16* __restrict__ x, int T, int tpad, int K, int ldx) {
    pdl_grid_sync();
    const int units = tpad * (K / 8);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < units; i += gridDim.x * blockDim.x) permute_x_unit(xp, x, i, T, K, ldx);
}

// One warp: MT tiles of 16 rows x NT*8 tokens over the groups kpart, kpart+ksplit, ... of the row's K.
// Tile mt covers rows tile_row0[mt] .. +15 (relative to Wp / S); rows >= rows_valid[mt] read as zero.
// `tok[nt]` is the activation row (in the permuted copy) that this lane supplies for column g of n-tile nt.
template <int MT, int NT>
__device__ __forceinline__ void warp_rows_times_tokens(float (&acc)[MT][NT][4], const uint8_t* __restrict__ Wp,
                                                       const uint8_t* __restrict__ S, size_t w_stride, size_t s_stride,
                                                       const int (&tile_row0)[MT], const int (&rows_valid)[MT], int K,
                                                       const uint4* __restrict__ xp, const int (&tok)[NT], int kpart, int ksplit) {
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
            const int ra = tile_row0[mt] + g, rb = ra + 8;
            if (group < G && g < rows_valid[mt]) {
                a0[mt] = ldg_nc_16(Wp + (size_t)ra * w_stride + (kk >> 1));
                b0[mt] = *reinterpret_cast<const uint16_t*>(S + (size_t)ra * s_stride + (kk >> 4));
            }
            if (group < G && g + 8 < rows_valid[mt]) {
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
            const uint4* xr = xp + ((size_t)tok[nt] * G + group) * 16 + c;
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
    // this block's weight rows (8 / ksplit tiles of MT*16 features, all of K) and their block scales
    PDL_ENTRY_WITH_PREFETCH({
        const int first = blockIdx.x * (8 / ksplit) * MT * 16;
        if (first < N) {
            const int rows = min((8 / ksplit) * MT * 16, N - first);
            prefetch_l2_rows(Wp + (size_t)first * (K / 2), rows, (size_t)K / 2);
            prefetch_l2_rows(S + (size_t)first * (K / 16), rows, (size_t)K / 16);
        }
    });
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
    if (n0 < N) {
        int row0[MT], valid[MT], tok[NT];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) { row0[mt] = mt * 16; valid[mt] = min(16, N - n0 - mt * 16); }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) tok[nt] = nt * 8 + g;
        warp_rows_times_tokens<MT, NT>(acc, Wp + (size_t)n0 * (K / 2), S + (size_t)n0 * (K / 16), K / 2, K / 16, row0, valid, K,
                                       xp, tok, kpart, ksplit);
    }
    pdl_trigger_late();
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
    const uint32_t ptag = use_push ? push_tag(push) : 0u;
    for (int i = threadIdx.x; i < tiles_per_block * TOK * ROWS; i += blockDim.x) {
        const int tl = i / (TOK * ROWS), rem = i % (TOK * ROWS), tok = rem / ROWS, r = rem % ROWS;
        const int n = (blockIdx.x * tiles_per_block + tl) * ROWS + r;
        if (tok < T && n < N) {
            float v = 0.f;
            for (int kp = 0; kp < ksplit; ++kp) v += red[(size_t)(tl * ksplit + kp) * (TOK * ROWS) + rem];
            v *= gs;
            if (use_push) {
                // fused all-reduce, producer side: the partial goes to every rank's receive slot
                push_store_all(push, tok, n, v, ptag);
            } else if (out_f32) ((float*)y)[(size_t)tok * N + n] = v;
            else ((bf16*)y)[(size_t)tok * N + n] = __float2bfloat16(v);
        }
    }
}

template <int MT, int NT>
int launch_linear(void* y, const void* x, void* xp, const void* Wp, const void* S, const void* g, int T, int N, int K, int ldx,
                  int out_f32, const PushCtx* push, cudaStream_t s) {
    constexpr int ROWS = MT * 16, TOK = NT * 8;
    const int units = TOK * (K / 8);
    // x == nullptr: the producer of the activations already wrote the permuted copy into xp
    if (x != nullptr) sl_launch(permute_x_kernel, (units + 255) / 256, 256, 0, s, (uint4*)xp, (const bf16*)x, T, TOK, K, ldx);
    int ksplit = 8;
    while (ksplit > 1 && K / 128 < ksplit) ksplit >>= 1;
    // few rows: keep the reduction split so that there are enough blocks to fill the machine
    const int tiles = (N + ROWS - 1) / ROWS;
    const int tiles_per_block = 8 / ksplit;
    auto kern = linear_nvfp4_mma_kernel<MT, NT>;
    const size_t smem = (size_t)8 * TOK * ROWS * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sl_launch(kern, (tiles + tiles_per_block - 1) / tiles_per_block, 256, smem, s, y, (const uint4*)xp, (const uint8_t*)Wp,
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

// xp = permuted f16 copy of x[T, K] (bf16, row stride ldx), rows T .. ceil(T/8)*8 - 1 zero.  K % 128 == 0, ldx % 8 == 0.
SL_API int sl_permute_x(void* xp, const void* x, int T, int K, int ldx, cudaStream_t s) {
    if (T == 0) return 0;
    if (K % 128 != 0 || ldx % 8 != 0) return -1;
    const int tpad = (T + 7) / 8 * 8, units = tpad * (K / 8);
    sl_launch(permute_x_kernel, (units + 255) / 256, 256, 0, s, (uint4*)xp, (const bf16*)x, T, tpad, K, ldx);
    return (int)cudaGetLastError();
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

// ======================================================================================================
// Decode-time MoE on the same weight-streaming scheme.  Routes (token, choice) that share an expert are
// grouped into work items of up to 8 activation rows, so an expert's weights are read once per step no
// matter how many tokens chose it.  Reference: `nvfp4_mul_mat_id_kernel` / `nvfp4_down_reduce_kernel`
// (`csrc/glm_gemv.cu:738-990, 1291-1375`) and the hybrid plan of `csrc/glm_mma_moe_coop.cu:43`.
//   plan      : routes -> items {expert, up to 8 routes}
//   gate/up   : act[route, :] = silu(g13[e,0] W1_e x_t) * (g13[e,1] W3_e x_t), written as f16 in operand order
//   down      : y_route[route, :] = g2[e] W2_e act[route, :]
//   reduce    : out[t, :] = sum_j wt[t,j] y_route[t*k+j, :] + y_route[shared(t), :]  (fp32, or pushed to peers)
namespace {

constexpr int kItemRoutes = 8;

struct MoePlanView {
    int* item_expert;      // [max_items]   local expert index, or -1 for the shared expert
    int* item_routes;      // [max_items][8] route ids (-1 padded)
    int* num_items;        // [1]
};

// ---- router GEMV + routing + plan (+ activation staging) in one launch ---------------------------------------
// grid (E/ROWS): a block multiplies ROWS (4 or 2) router rows by every token.  Warp w takes the 256-wide K steps w, w+8, ...
// of those rows (the rows of its first three steps are in registers before the kernel waits for its predecessor: the
// weights do not depend on it), reads the tokens' values straight from global memory, folds the lanes' partial sums
// with one transposing butterfly (31 shuffles for 32 sums) and meets the other warps in shared memory in a fixed
// order, so every rank computes bit-identical logits.  The block that finishes last (ticket counter) routes every
// token (one warp per token) and builds the work-item plan; all blocks share the conversion of the activations to the
// fragment order of the expert kernels.  Replaces the reference's router GEMV + `route_top8` + host-side plan
// (`csrc/glm_gemv.cu:1642`, `csrc/glm_ops.cu:2343`).
struct RouterFusedParams {
    const bf16* x; int ldx;                 // [T, H]
    const bf16* router_w;                   // [E, H]
    const float* bias;                      // [E] or null
    int T, H, E, top_k, n_group, topk_group, norm;
    float scale;
    float* logits;                          // [T][E] scratch
    unsigned int* counter;                  // zero before the first use; the kernel leaves it zero
    int* ids; float* wts;                   // [T, top_k]
    MoePlanView pv;
    int expert_offset, num_local, has_shared, max_items;
    uint4* xp; int tpad;                    // fragment-ordered copy of x to write (null: the caller has one)
};

// Sums v[i] over the 32 lanes for 32 values at once: afterwards lane l holds the total of v[l] in v[0].
__device__ __forceinline__ void warp_transpose_sum32(float (&v)[32]) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int o = 16, n = 32; o > 0; o >>= 1, n >>= 1) {
        const bool hi = lane & o;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
            const float a = v[i], b = v[i + n / 2];
            v[i] = (hi ? b : a) + __shfl_xor_sync(0xffffffffu, hi ? a : b, o);
        }
    }
}

// Plan for n = T * top_k <= 512 routes by one block of 256 threads in a few steps: the rank of a route among the
// routes of its expert comes from a warp match plus per-warp counts, the leaders of each chunk of 8 claim item slots
// in route order (so the plan does not depend on thread timing), members look their item up in a table.
// `sh`: (13 * E + 16) ints of shared memory; `ids` may be shared or global.
__device__ void moe_plan_fast(MoePlanView pv, const int* ids, int T, int top_k, int expert_offset, int num_local,
                              int has_shared, int max_items, int* sh) {
    const int n = T * top_k, E = num_local;
    int* cnt = sh;                                 // [8][E] routes of expert e in warp w of the current pass
    int* run = cnt + 8 * E;                        // [E] routes of expert e in earlier passes
    int* slot_tab = run + E;                       // [E][4] item of chunk c of expert e
    __shared__ int s_items;
    __shared__ int wcnt[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < 9 * E; i += 256) sh[i] = 0;
    if (tid == 0) s_items = 0;
    __syncthreads();
    for (int base = 0; base < n; base += 256) {
        const int r = base + tid;
        int e = -1;
        if (r < n) {
            const int le = ids[r] - expert_offset;
            e = (le >= 0 && le < num_local) ? le : -1;
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
        const bool leader = before >= 0 && (before % kItemRoutes) == 0;
        const unsigned m = __ballot_sync(0xffffffffu, leader);
        if (lane == 0) wcnt[warp] = __popc(m);
        __syncthreads();
        int slot = s_items, total = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            if (w < warp) slot += wcnt[w];
            total += wcnt[w];
        }
        slot += __popc(m & ((1u << lane) - 1));
        if (leader) {
            if (slot < max_items) { pv.item_expert[slot] = e; pv.item_routes[slot * kItemRoutes] = r; }
            if (before / kItemRoutes < 4) slot_tab[e * 4 + before / kItemRoutes] = slot;
        }
        __syncthreads();
        if (before >= 0 && !leader && before / kItemRoutes < 4) {
            const int it = slot_tab[e * 4 + before / kItemRoutes];
            if (it < max_items) pv.item_routes[it * kItemRoutes + before % kItemRoutes] = r;
        }
        if (tid == 0) s_items += total;
        __syncthreads();
        if (base + 256 < n) {
            for (int i = tid; i < E; i += 256) {
                int c = 0;
#pragma unroll
                for (int w = 0; w < 8; ++w) { c += cnt[w * E + i]; cnt[w * E + i] = 0; }
                run[i] += c;
            }
            __syncthreads();
        }
    }
    if (tid == 0) {
        int items = s_items;
        if (has_shared) {
            for (int t0 = 0; t0 < T; t0 += kItemRoutes) {
                if (items < max_items) {
                    pv.item_expert[items] = -1;
                    for (int q = 0; q < kItemRoutes && t0 + q < T; ++q) pv.item_routes[items * kItemRoutes + q] = n + t0 + q;
                }
                ++items;
            }
        }
        *pv.num_items = items < max_items ? items : max_items;
    }
}

__global__ void __launch_bounds__(256) moe_plan_kernel(MoePlanView pv, const int* __restrict__ ids, int T, int top_k,
                                                       int expert_offset, int num_local, int has_shared, int max_items) {
    pdl_grid_sync();
    extern __shared__ int sh[];
    for (int i = threadIdx.x; i < max_items * kItemRoutes; i += 256) pv.item_routes[i] = -1;
    __syncthreads();
    moe_plan_fast(pv, ids, T, top_k, expert_offset, num_local, has_shared, max_items, sh);
}

template <int PER, int ROWS>
__global__ void __launch_bounds__(256) router_route_plan_kernel(RouterFusedParams p) {
    constexpr int TG = 32 / ROWS;            // tokens per pass: ROWS x TG sums fill one transposing reduction
    extern __shared__ int dyn[];             // phase 1: [8 warps][32] partial sums; phase 2: plan tables + ids
    __shared__ int s_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int e0 = blockIdx.x * ROWS;
    const int steps = p.H / 256;
    constexpr int NPRE = 3;
    uint4 wv[NPRE][ROWS];
#pragma unroll
    for (int r = 0; r < NPRE; ++r) {
        const int st = r * 8 + warp;
#pragma unroll
        for (int j = 0; j < ROWS; ++j)
            wv[r][j] = (st < steps && e0 + j < p.E) ? ldg_nc_16(p.router_w + (size_t)(e0 + j) * p.H + st * 256 + lane * 8)
                                                    : make_uint4(0, 0, 0, 0);
    }
    pdl_grid_sync();
    // the plan's route table starts empty; the last block fills it after the ticket
    for (int i = blockIdx.x * 256 + tid; i < p.max_items * kItemRoutes; i += gridDim.x * 256) p.pv.item_routes[i] = -1;
    float* red = reinterpret_cast<float*>(dyn);
    for (int t0 = 0; t0 < p.T; t0 += TG) {
        float acc[32];                       // [ROWS][TG]
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = 0.f;
        auto round = [&](const uint4 (&wr)[ROWS], int st) {
            float wf[ROWS][8];
#pragma unroll
            for (int j = 0; j < ROWS; ++j) {
                const float2 a = bf162_to_f2(wr[j].x), b = bf162_to_f2(wr[j].y), c = bf162_to_f2(wr[j].z), d = bf162_to_f2(wr[j].w);
                wf[j][0] = a.x; wf[j][1] = a.y; wf[j][2] = b.x; wf[j][3] = b.y; wf[j][4] = c.x; wf[j][5] = c.y; wf[j][6] = d.x; wf[j][7] = d.y;
            }
#pragma unroll
            for (int h = 0; h < TG / 8; ++h) {    // eight tokens at a time: 8 loads in flight
                if (t0 + h * 8 >= p.T) break;
                uint4 xv[8];
#pragma unroll
                for (int t = 0; t < 8; ++t)
                    xv[t] = t0 + h * 8 + t < p.T
                                ? *reinterpret_cast<const uint4*>(p.x + (size_t)(t0 + h * 8 + t) * p.ldx + st * 256 + lane * 8)
                                : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    const float2 xa = bf162_to_f2(xv[t].x), xb = bf162_to_f2(xv[t].y), xc = bf162_to_f2(xv[t].z), xd = bf162_to_f2(xv[t].w);
#pragma unroll
                    for (int j = 0; j < ROWS; ++j)
                        acc[j * TG + h * 8 + t] += wf[j][0] * xa.x + wf[j][1] * xa.y + wf[j][2] * xb.x + wf[j][3] * xb.y +
                                                   wf[j][4] * xc.x + wf[j][5] * xc.y + wf[j][6] * xd.x + wf[j][7] * xd.y;
                }
            }
        };
#pragma unroll
        for (int r = 0; r < NPRE; ++r)
            if (r * 8 + warp < steps) round(wv[r], r * 8 + warp);
        for (int r = NPRE; r * 8 + warp < steps; ++r) {
            const int st = r * 8 + warp;
            uint4 wr[ROWS];
#pragma unroll
            for (int j = 0; j < ROWS; ++j)
                wr[j] = e0 + j < p.E ? ldg_nc_16(p.router_w + (size_t)(e0 + j) * p.H + st * 256 + lane * 8) : make_uint4(0, 0, 0, 0);
            round(wr, st);
        }
        warp_transpose_sum32(acc);
        __syncthreads();                     // the previous token group's sums have been read
        red[warp * 32 + lane] = acc[0];
        __syncthreads();
        if (tid < 32) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) v += red[w * 32 + tid];
            const int j = tid / TG, t = t0 + tid % TG;
            if (t < p.T && e0 + j < p.E) p.logits[(size_t)t * p.E + e0 + j] = v;
        }
    }
    if (p.xp != nullptr) {
        const int units = p.tpad * (p.H / 8);
        for (int i = blockIdx.x * 256 + tid; i < units; i += gridDim.x * 256) permute_x_unit(p.xp, p.x, i, p.T, p.H, p.ldx);
    }
    // ---- last block to finish takes over ----
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int ticket = atomicAdd(p.counter, 1u);
        s_last = ticket == gridDim.x - 1;
        if (s_last) *p.counter = 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    int* s_ids = dyn + 13 * p.num_local + 16;
    // warp w routes tokens w, w+8, w+16, w+24 together (their shuffle chains interleave)
    if (warp < p.T) {
        float lg[4][PER];
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            const int t = min(warp + 8 * n, p.T - 1);
#pragma unroll
            for (int i = 0; i < PER; ++i) lg[n][i] = lane * PER + i < p.E ? __ldcg(p.logits + (size_t)t * p.E + lane * PER + i) : 0.f;
        }
        int id[4];
        float w[4];
        if (p.T > 8) {
            route_warp_n<PER, 4>(lg, p.bias, p.E, p.top_k, p.n_group, p.topk_group, p.norm, p.scale, id, w);
        } else {
            route_warp<PER>(lg[0], p.bias, p.E, p.top_k, p.n_group, p.topk_group, p.norm, p.scale, id[0], w[0]);
        }
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            const int t = warp + 8 * n;
            if (t < p.T && lane < p.top_k) {
                p.ids[(size_t)t * p.top_k + lane] = id[n];
                p.wts[(size_t)t * p.top_k + lane] = w[n];
                s_ids[t * p.top_k + lane] = id[n];
            }
        }
    }
    __syncthreads();
    moe_plan_fast(p.pv, s_ids, p.T, p.top_k, p.expert_offset, p.num_local, p.has_shared, p.max_items, dyn);
}

struct MoeGroupedParams {
    const int* item_expert; const int* item_routes; const int* num_items;
    int T, top_k, H, I;
    const uint8_t *w13, *s13; const float* g13;        // [E, 2I, H/2], [E, 2I, H/16], [E, 2]
    const uint8_t *sw13, *ss13; const float* sg13;     // shared stack or null
    const uint8_t *w2, *s2; const float* g2;           // [E, H, I/2], [E, H, I/16], [E]
    const uint8_t *sw2, *ss2; const float* sg2;
    const uint4* xp;                                   // permuted x, [Tpad rows][H]
    uint4* act_perm;                                   // permuted act, [routes_pad][I] f16
    float* y_route;                                    // [routes, H]
};

// grid (ceil(I/16 / tiles_per_block), max_items).  Warp = (tile, kpart): gate rows i0..i0+15 and up rows I+i0.. .
__global__ void __launch_bounds__(256) moe_gate_up_mma_kernel(MoeGroupedParams p, int ksplit) {
    pdl_grid_sync();
    extern __shared__ float red[];                 // [8 warps][2 tiles][8 tok][16 rows]
    const int item = blockIdx.y;
    if (item >= *p.num_items) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int tiles_per_block = 8 / ksplit, tile = warp / ksplit, kpart = warp % ksplit;
    const int i0 = (blockIdx.x * tiles_per_block + tile) * 16;
    const int e = p.item_expert[item];
    const uint8_t* W = e < 0 ? p.sw13 : p.w13 + (size_t)e * 2 * p.I * (p.H / 2);
    const uint8_t* S = e < 0 ? p.ss13 : p.s13 + (size_t)e * 2 * p.I * (p.H / 16);
    const float* G = e < 0 ? p.sg13 : p.g13 + (size_t)e * 2;
    const int n_routed = p.T * p.top_k;
    const int route_g = p.item_routes[item * kItemRoutes + g];
    int tok[1];
    tok[0] = route_g < 0 ? 0 : (route_g < n_routed ? route_g / p.top_k : route_g - n_routed);
    float acc[2][1][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) acc[mt][0][0] = acc[mt][0][1] = acc[mt][0][2] = acc[mt][0][3] = 0.f;
    if (i0 < p.I) {
        const int row0[2] = {i0, p.I + i0};
        const int v = min(16, p.I - i0);
        const int valid[2] = {v, v};
        warp_rows_times_tokens<2, 1>(acc, W, S, p.H / 2, p.H / 16, row0, valid, p.H, p.xp, tok, kpart, ksplit);
    }
    float* mine = red + (size_t)warp * (2 * 8 * 16);
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
        mine[(mt * 8 + 2 * c) * 16 + g] = acc[mt][0][0];
        mine[(mt * 8 + 2 * c + 1) * 16 + g] = acc[mt][0][1];
        mine[(mt * 8 + 2 * c) * 16 + g + 8] = acc[mt][0][2];
        mine[(mt * 8 + 2 * c + 1) * 16 + g + 8] = acc[mt][0][3];
    }
    __syncthreads();
    const float gg = G[0], gu = G[1];
    const int Gd = p.I / 128;
    __half* act = reinterpret_cast<__half*>(p.act_perm);
    for (int idx = threadIdx.x; idx < tiles_per_block * 8 * 16; idx += blockDim.x) {
        const int tl = idx / 128, rem = idx % 128, slot = rem / 16, r = rem % 16;
        const int i = (blockIdx.x * tiles_per_block + tl) * 16 + r;
        const int route = p.item_routes[item * kItemRoutes + slot];
        if (route < 0 || i >= p.I) continue;
        float gs = 0.f, us = 0.f;
        for (int kp = 0; kp < ksplit; ++kp) {
            const float* w = red + (size_t)(tl * ksplit + kp) * (2 * 8 * 16);
            gs += w[(0 * 8 + slot) * 16 + r];
            us += w[(1 * 8 + slot) * 16 + r];
        }
        gs *= gg; us *= gu;
        const float a = gs / (1.f + __expf(-gs)) * us;
        const int w128 = i % 128, cc = w128 / 32, jj = (w128 % 32) / 8, ee = w128 % 8;
        act[((((size_t)route * Gd + i / 128) * 16 + jj * 4 + cc) * 8) + ee] = __float2half(a);
    }
}

// grid (ceil(H/16 / tiles_per_block), max_items).  B operand rows = the item's routes (their act rows).
__global__ void __launch_bounds__(256) moe_down_mma_kernel(MoeGroupedParams p, int ksplit) {
    pdl_grid_sync();
    extern __shared__ float red[];                 // [8 warps][8 tok][16 rows]
    const int item = blockIdx.y;
    if (item >= *p.num_items) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int tiles_per_block = 8 / ksplit, tile = warp / ksplit, kpart = warp % ksplit;
    const int n0 = (blockIdx.x * tiles_per_block + tile) * 16;
    const int e = p.item_expert[item];
    const uint8_t* W = e < 0 ? p.sw2 : p.w2 + (size_t)e * p.H * (p.I / 2);
    const uint8_t* S = e < 0 ? p.ss2 : p.s2 + (size_t)e * p.H * (p.I / 16);
    const float gs = e < 0 ? p.sg2[0] : p.g2[e];
    const int route_g = p.item_routes[item * kItemRoutes + g];
    int tok[1];
    tok[0] = route_g < 0 ? 0 : route_g;
    float acc[1][1][4] = {{{0.f, 0.f, 0.f, 0.f}}};
    if (n0 < p.H) {
        const int row0[1] = {n0};
        const int valid[1] = {min(16, p.H - n0)};
        warp_rows_times_tokens<1, 1>(acc, W, S, p.I / 2, p.I / 16, row0, valid, p.I, p.act_perm, tok, kpart, ksplit);
    }
    float* mine = red + (size_t)warp * (8 * 16);
    mine[(2 * c) * 16 + g] = acc[0][0][0];
    mine[(2 * c + 1) * 16 + g] = acc[0][0][1];
    mine[(2 * c) * 16 + g + 8] = acc[0][0][2];
    mine[(2 * c + 1) * 16 + g + 8] = acc[0][0][3];
    __syncthreads();
    for (int idx = threadIdx.x; idx < tiles_per_block * 8 * 16; idx += blockDim.x) {
        const int tl = idx / 128, rem = idx % 128, slot = rem / 16, r = rem % 16;
        const int n = (blockIdx.x * tiles_per_block + tl) * 16 + r;
        const int route = p.item_routes[item * kItemRoutes + slot];
        if (route < 0 || n >= p.H) continue;
        float v = 0.f;
        for (int kp = 0; kp < ksplit; ++kp) v += red[(size_t)(tl * ksplit + kp) * (8 * 16) + rem];
        p.y_route[(size_t)route * p.H + n] = v * gs;
    }
}

// out[t, n] = sum_j wt[t,j] * y_route[t*k+j, n] (local experts only) + y_route[T*k + t, n]
__global__ void moe_route_reduce_kernel(const float* __restrict__ y_route, const int* __restrict__ ids, const float* __restrict__ wts,
                                        int T, int top_k, int H, int expert_offset, int num_local, int has_shared,
                                        float* __restrict__ out, int use_push, PushCtx push) {
    pdl_grid_sync();
    const int t = blockIdx.y;
    const uint32_t ptag = use_push ? push_tag(push) : 0u;
    for (int n = blockIdx.x * blockDim.x + threadIdx.x; n < H; n += gridDim.x * blockDim.x) {
        float v = 0.f;
        for (int j = 0; j < top_k; ++j) {
            const int e = ids[t * top_k + j] - expert_offset;
            if (e >= 0 && e < num_local) v += wts[t * top_k + j] * y_route[(size_t)(t * top_k + j) * H + n];
        }
        if (has_shared) v += y_route[(size_t)(T * top_k + t) * H + n];
        if (use_push) {
            push_store_all(push, t, n, v, ptag);
        } else {
            out[(size_t)t * H + n] = v;
        }
    }
}

int pick_ksplit(int K, int min_groups_per_warp) {
    int ks = 8;
    while (ks > 1 && (K / 128) / ks < min_groups_per_warp) ks >>= 1;
    return ks;
}

}  // namespace

// out[t, :] = sum_j wts[t, j] * y_route[t * top_k + j, :] (+ y_route[T * top_k + t, :] for the shared expert), fp32, or
// pushed to every rank's receive slot (producer half of the fused all-reduce): the last stage of the decode MoE layer on
// its own, for callers that computed `y_route` with other kernels (the block-scaled FP4 GEMMs).
SL_API int sl_moe_route_reduce(const void* y_route, const void* ids, const void* wts, int T, int top_k, int H, int expert_offset,
                               int num_local, int has_shared, void* out, const PushCtx* push, cudaStream_t s) {
    if (T == 0) return 0;
    if (push != nullptr && (T > push->slot_rows || H > push->row_len)) return -1;
    if (push == nullptr && out == nullptr) return -1;
    sl_launch(moe_route_reduce_kernel, dim3((H + 255) / 256, T), 256, 0, s, (const float*)y_route, (const int*)ids, (const float*)wts, T,
              top_k, H, expert_offset, num_local, has_shared, (float*)out, push ? 1 : 0, push ? *push : PushCtx{});
    return (int)cudaGetLastError();
}

struct MoeGroupedArgs {
    const void* x; int ldx;
    const void* ids; const void* wts;
    int T, top_k, H, I, expert_offset, num_local;
    const void *w13, *s13, *g13, *sw13, *ss13, *sg13;
    const void *w2, *s2, *g2, *sw2, *ss2, *sg2;
    // caller-owned scratch
    void* xp;            // f16 [ceil(T/8)*8, H]
    void* act_perm;      // f16 [routes + 8, I]
    void* y_route;       // f32 [routes, H]
    void* plan;          // int32 [max_items * 9 + 1]
    int max_items;
    void* out;           // f32 [T, H] (ignored when pushing)
    int xp_ready;        // the activations' producer already wrote the permuted copy into xp
};

// Optional router stage: with it the layer starts from the normed hidden state alone and writes the chosen
// experts and weights to a->ids / a->wts itself.
struct MoeRouterArgs {
    const void* router_w;    // bf16 [E, H]
    const void* bias;        // f32 [E] or null
    int E, n_group, topk_group, norm;
    float scale;
    void* slabs;             // f32 [T, E] scratch (the logits)
    void* counter;           // u32, zero before the first use (the kernel leaves it zero)
};

template <int PER>
static void launch_router(const RouterFusedParams& rp, size_t smem, cudaStream_t s) {
    // few tokens: 4 rows per block (8-token passes); more: 2 rows per block (16-token passes, twice the blocks)
    if (rp.T <= 8) {
        auto kern = router_route_plan_kernel<PER, 4>;
        sl_launch(kern, dim3((rp.E + 3) / 4), 256, smem, s, rp);
    } else {
        auto kern = router_route_plan_kernel<PER, 2>;
        sl_launch(kern, dim3((rp.E + 1) / 2), 256, smem, s, rp);
    }
}

// Decode-time MoE layer for T <= 32 tokens: (router, routing,) plan, gate/up, down, weighted reduce (optionally
// pushed to every rank's receive slot as the producer half of the fused all-reduce).  H % 128 == 0, I % 128 == 0;
// with a router stage also H % 256 == 0.
SL_API int sl_moe_grouped_mma(const MoeGroupedArgs* a, const MoeRouterArgs* r, const PushCtx* push, cudaStream_t s) {
    if (a->T == 0) return 0;
    if (a->T > 32 || a->H % 128 != 0 || a->I % 128 != 0 || a->ldx % 8 != 0 || a->T * a->top_k > 480) return -1;
    if (push != nullptr && (a->T > push->slot_rows || a->H > push->row_len)) return -1;
    const int has_shared = a->sw13 != nullptr;
    const int n_routed = a->T * a->top_k;
    int* plan = (int*)a->plan;
    MoePlanView pv{plan, plan + a->max_items, plan + a->max_items * (1 + kItemRoutes)};
    bool xp_done = false;
    if (r != nullptr) {
        if (a->H % 256 != 0 || r->E > 512 || a->top_k > 32 || r->n_group > 32 || r->n_group < 1 || r->E % r->n_group != 0) return -1;
        int PER = 1;
        while (PER * 32 < r->E) PER <<= 1;
        if (r->n_group > 1) {
            const int gsz = r->E / r->n_group;
            if (gsz % PER != 0) return -1;                   // a group must be a run of whole lanes
            const int lpg = gsz / PER;
            if (lpg & (lpg - 1)) return -1;
        }
        const int tpad8 = (a->T + 7) / 8 * 8;
        RouterFusedParams rp{(const bf16*)a->x, a->ldx, (const bf16*)r->router_w, (const float*)r->bias, a->T, a->H, r->E,
                             a->top_k, r->n_group, r->topk_group, r->norm, r->scale, (float*)r->slabs,
                             (unsigned int*)r->counter, (int*)a->ids, (float*)a->wts, pv, a->expert_offset, a->num_local,
                             has_shared, a->max_items, a->xp_ready ? nullptr : (uint4*)a->xp, tpad8};
        size_t smem = (size_t)8 * 32 * sizeof(float);
        const size_t smem2 = (size_t)(13 * a->num_local + 16 + n_routed) * sizeof(int);
        if (smem2 > smem) smem = smem2;
        if (smem > 48 * 1024 || a->num_local < 1) return -1;
        switch (PER) {
            case 1: launch_router<1>(rp, smem, s); break;
            case 2: launch_router<2>(rp, smem, s); break;
            case 4: launch_router<4>(rp, smem, s); break;
            case 8: launch_router<8>(rp, smem, s); break;
            default: launch_router<16>(rp, smem, s); break;
        }
        xp_done = true;
    } else {
        const size_t smem = (size_t)(13 * a->num_local + 16) * sizeof(int);
        if (smem > 48 * 1024 || a->num_local < 1) return -1;
        sl_launch(moe_plan_kernel, 1, 256, smem, s, pv, (const int*)a->ids, a->T, a->top_k,
                  a->expert_offset, a->num_local, has_shared, a->max_items);
    }
    if (a->w13 == nullptr) return (int)cudaGetLastError();      // routing + plan only (the expert GEMMs run elsewhere)
    const int tpad = (a->T + 7) / 8 * 8;
    const int units = tpad * (a->H / 8);
    if (!a->xp_ready && !xp_done)
        sl_launch(permute_x_kernel, (units + 255) / 256, 256, 0, s, (uint4*)a->xp, (const bf16*)a->x, a->T, tpad, a->H, a->ldx);
    MoeGroupedParams p{pv.item_expert, pv.item_routes, pv.num_items, a->T, a->top_k, a->H, a->I,
                       (const uint8_t*)a->w13, (const uint8_t*)a->s13, (const float*)a->g13,
                       (const uint8_t*)a->sw13, (const uint8_t*)a->ss13, (const float*)a->sg13,
                       (const uint8_t*)a->w2, (const uint8_t*)a->s2, (const float*)a->g2,
                       (const uint8_t*)a->sw2, (const uint8_t*)a->ss2, (const float*)a->sg2,
                       (const uint4*)a->xp, (uint4*)a->act_perm, (float*)a->y_route};
    {
        const int ks = pick_ksplit(a->H, 4), tpb = 8 / ks, tiles = (a->I + 15) / 16;
        const size_t smem = (size_t)8 * 2 * 8 * 16 * sizeof(float);
        sl_launch(moe_gate_up_mma_kernel, dim3((tiles + tpb - 1) / tpb, a->max_items), 256, smem, s, p, ks);
    }
    {
        const int ks = pick_ksplit(a->I, 4), tpb = 8 / ks, tiles = (a->H + 15) / 16;
        const size_t smem = (size_t)8 * 8 * 16 * sizeof(float);
        sl_launch(moe_down_mma_kernel, dim3((tiles + tpb - 1) / tpb, a->max_items), 256, smem, s, p, ks);
    }
    int bx = (a->H + 255) / 256;
    sl_launch(moe_route_reduce_kernel, dim3(bx, a->T), 256, 0, s, (const float*)a->y_route, (const int*)a->ids, (const float*)a->wts, a->T,
                                                          a->top_k, a->H, a->expert_offset, a->num_local, has_shared,
                                                          (float*)a->out, push ? 1 : 0, push ? *push : PushCtx{});
    return (int)cudaGetLastError();
}
