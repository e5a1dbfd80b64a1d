// Expert parallelism over NVLink peer memory: token dispatch and weighted combine around the block-scaled grouped GEMMs.
//
// Every rank is the *home* of a slice of the step's tokens and the *owner* of E / W experts.  One round:
//   1. home   routes its tokens, sorts its routes by (global) expert and pushes the per-expert counts to every rank
//   2. all    wait for the W count vectors; from them every rank derives, identically, where each (source rank, expert)
//             run of rows starts in its owner's expert-sorted receive buffer (and in the buffer's padded scale tiles)
//   3. home   dispatch: the 4-bit row of each routed token (codes, scale words, global scale) is stored straight into
//             the owner's receive buffer at its final sorted position, with {home rank, route slot} beside it;
//             the last block of the kernel publishes "my rows have landed" to every owner
//   4. owner  waits for the W dispatch flags, runs gate/up (SiLU * mul), re-quantisation and the down projection as
//             grouped NVFP4 GEMMs over the received rows (csrc/gemm_fp4_tcgen05.cu); the down GEMM's epilogue stores each
//             output row into the *home* rank's combine buffer at the route's slot (no local copy, no second pass)
//   5. owner  publishes "my results have landed"; home waits for W flags and sums its routes with the routing weights
// No host synchronisation, no data-dependent launch shape: buffer capacities are fixed upper bounds, the row counts live
// on the device, so the round can be captured in a CUDA graph.  Plain peer stores only (no multimem, no TMA multicast).
// Waits are bounded: on expiry a status word is written and the kernel returns.  Two rounds on the same buffers must be
// separated by a collective that every rank takes part in (the all-reduce that follows every MoE layer is one).
//
// The reference has no expert parallelism; its nearest pieces are the expert permute / un-permute kernels
// (`csrc/glm_mma_moe_coop.cu:155-262`, `csrc/glm_mma_moe.cu:415-470`).
#include <algorithm>

#include "common.cuh"

#define SL_EP_MAX_RANKS 8

struct EpCtx {
    int* counts[SL_EP_MAX_RANKS];          // on rank p: [W][E], row r = routes per global expert among rank r's home tokens
    uint32_t* flags[SL_EP_MAX_RANKS];      // on rank p: [3][W] epoch tags (counts, dispatch, combine) written by rank r
    uint8_t* recv_q[SL_EP_MAX_RANKS];      // [cap][K/2] received token rows, expert-sorted
    uint8_t* recv_sf[SL_EP_MAX_RANKS];     // their scale tiles [cap / bn + El][K/64][512]
    float* recv_g[SL_EP_MAX_RANKS];        // [cap]
    int2* recv_meta[SL_EP_MAX_RANKS];      // [cap] {home rank, route slot at home}
    bf16* comb[SL_EP_MAX_RANKS];           // [home_cap][H] expert outputs of this rank's routes
    uint32_t* epoch;                       // local: rounds completed
    uint32_t* done;                        // local: block tickets (zero between kernels)
    int* status;                           // {code, site, expected, seen}
    int rank, world, E, El, cap, home_cap, K, H, bn;
    uint32_t max_spins;
};

namespace {

__device__ __forceinline__ void ep_fail(const EpCtx& c, int site, int expected, int seen) {
    if (c.status != nullptr && atomicCAS(c.status, 0, 3) == 0) {
        c.status[1] = site; c.status[2] = expected; c.status[3] = seen;
    }
}

// counts of this rank's routes per global expert (differences of the local sort's offsets) -> every rank
__global__ void __launch_bounds__(1024) ep_counts_push_kernel(const EpCtx c, const int* __restrict__ offsets_local) {
    pdl_grid_sync();
    const uint32_t tag = *c.epoch + 1u;
    for (int e = threadIdx.x; e < c.E; e += blockDim.x) {
        const int n = offsets_local[e + 1] - offsets_local[e];
        for (int p = 0; p < c.world; ++p) c.counts[p][(size_t)c.rank * c.E + e] = n;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < c.world) st_relaxed_sys_u32(c.flags[threadIdx.x] + 0 * c.world + c.rank, tag);
}

// One block.  Waits for every rank's counts, then lays out every owner's receive buffer:
//   rows of owner o: experts o*El .. in order, inside an expert the source ranks in order
//   my_offsets[El + 1], my_pad[El + 1]: this rank's own expert groups (rows, and rows padded to multiples of bn)
//   dest_row[E], dest_prow[E]: where this rank's rows for global expert e start at e's owner
__global__ void __launch_bounds__(1024) ep_plan_kernel(const EpCtx c, int* __restrict__ my_offsets, int* __restrict__ my_pad,
                                                       int* __restrict__ dest_row, int* __restrict__ dest_prow) {
    pdl_grid_sync();
    __shared__ int tot[1024], before_me[1024], off[1025], padoff[1025];
    const uint32_t tag = *c.epoch + 1u;
    if ((int)threadIdx.x < c.world)
        if (!wait_flag_geq(c.flags[c.rank] + 0 * c.world + threadIdx.x, tag, c.max_spins, c.status, 40)) { /* status recorded */ }
    __syncthreads();
    const int* cnt = c.counts[c.rank];
    for (int e = threadIdx.x; e < c.E; e += blockDim.x) {
        int t = 0, b = 0;
        for (int r = 0; r < c.world; ++r) {
            const int n = cnt[(size_t)r * c.E + e];
            if (r < c.rank) b += n;
            t += n;
        }
        tot[e] = t;
        before_me[e] = b;
    }
    __syncthreads();
    // per owner: prefix over its El experts (thread o handles owner o)
    if ((int)threadIdx.x < c.world) {
        const int o = threadIdx.x;
        int run = 0, prun = 0;
        for (int el = 0; el < c.El; ++el) {
            const int e = o * c.El + el;
            off[e] = run; padoff[e] = prun;
            run += tot[e];
            prun += (tot[e] + c.bn - 1) / c.bn * c.bn;
        }
        if (run > c.cap) ep_fail(c, 41, c.cap, run);           // an owner's receive buffer would overflow
        if (o == c.rank) {
            my_offsets[c.El] = min(run, c.cap);
            my_pad[c.El] = prun;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < c.E; e += blockDim.x) {
        dest_row[e] = off[e] + before_me[e];
        dest_prow[e] = padoff[e] + before_me[e];
        if (e / c.El == c.rank) {
            my_offsets[e % c.El] = min(off[e], c.cap);
            my_pad[e % c.El] = padoff[e];
        }
    }
}

// One block per locally sorted route row m (grid >= 1).  q_tok / sf_tok / g_tok: this rank's home tokens quantised once
// (ungrouped scale tiles of `src_bn` rows).  order[m] = route (token * k + j), offsets_local [E + 1].
struct EpDispatchArgs {
    const uint8_t* q_tok; const uint8_t* sf_tok; const float* g_tok;
    const int* order; const int* offsets_local; const int* dest_row; const int* dest_prow;
    int n_routes, top_k, src_bn, tokens;
};

__global__ void __launch_bounds__(256) ep_dispatch_kernel(const EpCtx c, const EpDispatchArgs a) {
    pdl_grid_sync();
    const int m = blockIdx.x, ks = threadIdx.x;
    const int KT = c.K / 64;
    if (m < a.n_routes && ks < KT) {
        int lo = 0, hi = c.E;                              // expert of sorted row m: last e with offsets_local[e] <= m
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (__ldg(a.offsets_local + mid) <= m) lo = mid; else hi = mid;
        }
        // (rows behind the last local expert are routes to no expert of the model: none under EP, ids are global)
        const int e = lo, idx = m - __ldg(a.offsets_local + e);
        const int owner = e / c.El;
        const int row = __ldg(a.dest_row + e) + idx, prow = __ldg(a.dest_prow + e) + idx;
        const int route = __ldg(a.order + m), tok = route / a.top_k;
        if (row < c.cap && tok < a.tokens) {
            const uint4* qs = reinterpret_cast<const uint4*>(a.q_tok + (size_t)tok * (c.K / 2) + (size_t)ks * 32);
            uint4* qd = reinterpret_cast<uint4*>(c.recv_q[owner] + (size_t)row * (c.K / 2) + (size_t)ks * 32);
            qd[0] = __ldg(qs); qd[1] = __ldg(qs + 1);
            const int st = tok / a.src_bn, sr = tok % a.src_bn;
            const uint32_t sc = __ldg(reinterpret_cast<const uint32_t*>(a.sf_tok + ((size_t)st * KT + ks) * 512 + (sr % 32) * 16 + (sr / 32) * 4));
            const int tile = prow / c.bn, r = prow % c.bn;
            *reinterpret_cast<uint32_t*>(c.recv_sf[owner] + ((size_t)tile * KT + ks) * 512 + (r % 32) * 16 + (r / 32) * 4) = sc;
            if (ks == 0) {
                c.recv_g[owner][row] = __ldg(a.g_tok + tok);
                c.recv_meta[owner][row] = make_int2(c.rank, route);
            }
        }
    }
    // "my rows have landed": every block orders its stores, the last one to finish tells the owners
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t ticket = atomicAdd(c.done, 1u);
        if (ticket == gridDim.x - 1) {
            *c.done = 0u;
            __threadfence_system();
            const uint32_t tag = *c.epoch + 1u;
            for (int p = 0; p < c.world; ++p) st_relaxed_sys_u32(c.flags[p] + 1 * c.world + c.rank, tag);
        }
    }
}

// kind 1: all dispatches into this rank have landed; kind 2: all results for this rank's routes have landed
__global__ void ep_wait_kernel(const EpCtx c, int kind) {
    pdl_grid_sync();
    const uint32_t tag = *c.epoch + 1u;
    if ((int)threadIdx.x < c.world) wait_flag_geq(c.flags[c.rank] + kind * c.world + threadIdx.x, tag, c.max_spins, c.status, 42 + kind);
}

// after the down GEMM (whose epilogue stored into the home ranks' combine buffers): tell every home rank
__global__ void ep_signal_kernel(const EpCtx c, int kind) {
    pdl_grid_sync();
    __threadfence_system();
    const uint32_t tag = *c.epoch + 1u;
    if ((int)threadIdx.x < c.world) st_relaxed_sys_u32(c.flags[threadIdx.x] + kind * c.world + c.rank, tag);
}

// out[t, n] (+)= sum_j wts[t, j] * comb[t * k + j, n]; the last block closes the round (epoch + 1)
__global__ void __launch_bounds__(256) ep_reduce_kernel(const EpCtx c, float* __restrict__ out, int ldo, const float* __restrict__ wts,
                                                        int tokens, int top_k, int accumulate) {
    pdl_grid_sync();
    const int t = blockIdx.y;
    const bf16* rows = c.comb[c.rank];
    for (int n = (blockIdx.x * blockDim.x + threadIdx.x) * 8; n < c.H; n += gridDim.x * blockDim.x * 8) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = accumulate ? out[(size_t)t * ldo + n + i] : 0.f;
        for (int j = 0; j < top_k; ++j) {
            const float w = wts[t * top_k + j];
            const uint4 v = *reinterpret_cast<const uint4*>(rows + (size_t)(t * top_k + j) * c.H + n);
            const float2 a = bf162_to_f2(v.x), b = bf162_to_f2(v.y), d = bf162_to_f2(v.z), e = bf162_to_f2(v.w);
            acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * b.x; acc[3] += w * b.y;
            acc[4] += w * d.x; acc[5] += w * d.y; acc[6] += w * e.x; acc[7] += w * e.y;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) out[(size_t)t * ldo + n + i] = acc[i];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t ticket = atomicAdd(c.done, 1u);
        if (ticket == gridDim.x * gridDim.y - 1) {
            *c.done = 0u;
            atomicAdd(c.epoch, 1u);
        }
    }
}

__global__ void ep_close_round_kernel(const EpCtx c) {
    pdl_grid_sync();
    if (threadIdx.x == 0) atomicAdd(c.epoch, 1u);
}

}  // namespace

SL_API int sl_ep_counts_push(const EpCtx* c, const void* offsets_local, cudaStream_t s) {
    if (c->E > 1024 || c->world > SL_EP_MAX_RANKS || c->E % c->world != 0) return -1;
    sl_launch(ep_counts_push_kernel, 1, 1024, 0, s, *c, (const int*)offsets_local);
    return (int)cudaGetLastError();
}

SL_API int sl_ep_plan(const EpCtx* c, void* my_offsets, void* my_pad, void* dest_row, void* dest_prow, cudaStream_t s) {
    if (c->E > 1024) return -1;
    sl_launch(ep_plan_kernel, 1, 1024, 0, s, *c, (int*)my_offsets, (int*)my_pad, (int*)dest_row, (int*)dest_prow);
    return (int)cudaGetLastError();
}

SL_API int sl_ep_dispatch(const EpCtx* c, const void* q_tok, const void* sf_tok, const void* g_tok, const void* order,
                          const void* offsets_local, const void* dest_row, const void* dest_prow, int n_routes, int top_k, int src_bn,
                          int tokens, cudaStream_t s) {
    if (c->K % 64 != 0 || c->K > 16384) return -1;
    EpDispatchArgs a{(const uint8_t*)q_tok, (const uint8_t*)sf_tok, (const float*)g_tok, (const int*)order, (const int*)offsets_local,
                     (const int*)dest_row, (const int*)dest_prow, n_routes, top_k, src_bn, tokens};
    sl_launch(ep_dispatch_kernel, n_routes > 0 ? n_routes : 1, (c->K / 64 + 31) / 32 * 32, 0, s, *c, a);
    return (int)cudaGetLastError();
}

SL_API int sl_ep_wait(const EpCtx* c, int kind, cudaStream_t s) {
    if (kind < 0 || kind > 2) return -1;
    sl_launch(ep_wait_kernel, 1, 32, 0, s, *c, kind);
    return (int)cudaGetLastError();
}

SL_API int sl_ep_signal(const EpCtx* c, int kind, cudaStream_t s) {
    if (kind < 0 || kind > 2) return -1;
    sl_launch(ep_signal_kernel, 1, 32, 0, s, *c, kind);
    return (int)cudaGetLastError();
}

// Weighted sum of this rank's routes into out [tokens, ldo] fp32 (rows = this rank's home tokens); ends the round.
SL_API int sl_ep_reduce(const EpCtx* c, void* out, int ldo, const void* wts, int tokens, int top_k, int accumulate, cudaStream_t s) {
    if (c->H % 8 != 0) return -1;
    if (tokens <= 0) {
        sl_launch(ep_close_round_kernel, 1, 32, 0, s, *c);
        return (int)cudaGetLastError();
    }
    const int bx = std::max(1, std::min(4, (c->H / 8 + 255) / 256));
    sl_launch(ep_reduce_kernel, dim3(bx, tokens), 256, 0, s, *c, (float*)out, ldo, (const float*)wts, tokens, top_k, accumulate);
    return (int)cudaGetLastError();
}
