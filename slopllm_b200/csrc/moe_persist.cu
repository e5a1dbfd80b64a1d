// Decode-time MoE layer (1..32 token rows) as ONE persistent kernel: router product, routing + work plan, grouped
// gate/up with SiLU * mul, grouped down projection and the routing-weighted sum (optionally stored into every rank's
// receive slot as the producer half of the fused all-reduce).
//
// The layer's work is a single ordered queue of tiles
//     [router tiles][shared-expert gate/up tiles][plan tile][routed gate/up tiles][down tiles][reduce tiles]
// that the thread blocks (one per SM) claim with an atomic counter.  A tile that needs the output of earlier tiles waits
// on a completion counter of those tiles.  Because a tile only ever waits for tiles that precede it in the queue, and a
// claimed tile is worked on at once, the kernel finishes with any number of resident blocks (no cooperative launch).
// Every wait is bounded: on expiry the block records a status and all blocks leave.
//
// Inside a block, warp 0 is the producer: it claims tiles one ahead of the consumers and streams each tile's weight rows
// into a ring of shared-memory stages with `cp.async.bulk` (mbarrier transaction counts), so the weights of a tile are in
// flight while it still waits for its activations and while the previous tile is being computed.  Warps 1..8 consume:
// NVFP4 codes are expanded to f16 in registers (x UE4M3 block scale) and multiplied with the (up to eight) activation
// rows of a work item by `mma.sync.m16n8k16`, exactly the arithmetic of `moe_gate_up_mma_kernel` / `moe_down_mma_kernel`
// (csrc/gemv_mma.cu), which this kernel replaces on the decode path.
//
// Reference counterpart: the five launches router GEMV + `route_top8` + `nvfp4_mul_mat_id_kernel` x2 +
// `nvfp4_down_reduce_kernel` (`csrc/glm_gemv.cu:738-990, 1291-1375`, `csrc/glm_ops.cu:2343`).
#include "push.cuh"
#include "route.cuh"
#include "tcgen05.cuh"
#include "w4_frag.cuh"

namespace {

constexpr int kStageBytes = 57344;
constexpr int kStages = 3;
constexpr int kConsumerWarps = 8;
constexpr int kConsumers = 32 * kConsumerWarps;
constexpr int kThreads = 32 + kConsumers;
constexpr int kItemRoutes = 8;
constexpr uint64_t kWaitLimitNs = 1000000000ull;              // every wait gives up after a second
constexpr int kTraceEntries = 96;                             // per block: {kind << 32 | item << 8 | blk, start, inputs ready, end}

enum TileKind : int { kRouter = 0, kGate = 1, kPlan = 2, kDown = 3, kReduce = 4, kExit = 5 };

// words of the `sync` array (all zero between launches)
enum SyncWord : int { kQueue = 0, kRouterDone = 1, kPlanDone = 2, kDownDone = 3, kExitCount = 4, kGateTotal = 5, kGateDone = 8 };

struct Work {
    int kind, item, expert, blk;
    int routes[kItemRoutes];
};

struct MoePersistParams {
    const bf16* x; int ldx;                 // [T, H] normed hidden rows (router input)
    const uint4* xp;                        // permuted f16 copy of x (see common.cuh)
    const bf16* router_w;                   // [E, H] or null (then `ids` / `wts` are inputs)
    const float* bias;
    int E, n_group, topk_group, norm;
    float scale;
    int T, top_k, H, I, expert_offset, num_local;
    const uint8_t *w13, *s13; const float* g13;        // [E, 2I, H/2], [E, 2I, H/16], [E, 2]
    const uint8_t *sw13, *ss13; const float* sg13;     // shared expert or null
    const uint8_t *w2, *s2; const float* g2;           // [E, H, I/2], [E, H, I/16], [E]
    const uint8_t *sw2, *ss2; const float* sg2;
    float* slabs;                           // [RK][T][E] partial router logits
    uint4* act_perm;                        // permuted f16 [routes + 8][I]
    float* y_route;                         // [routes][H]
    int* item_expert; int* item_routes; int* num_items;
    int* ids; float* wts;                   // [T, top_k]
    uint32_t* sync;                         // counters, see SyncWord
    int* status;                            // {code, site, expected, seen}
    float* out;                             // [T, H] fp32 (unused when pushing)
    int max_items;
    // tiling (filled by the host)
    int RK, KC;                             // router: K chunks, chunk length
    int n_router, n_shared_items;
    int gsub, TG;                           // gate/up: sub-tiles (8 columns) per tile, tiles per item
    int KSd, RTd, drep, dsub, TD;           // down: K splits, 16-row tiles per pass, passes per sub-tile, sub-tiles per tile, tiles per item
    int n_stages, xs_mode;                  // stages in use; T <= 8: token rows resident in shared memory
    int off_xs, off_scratch, off_plan, off_ctl;     // byte offsets of the shared-memory areas
    int NXB;                                // reduce: column blocks of 1024 per token
    int WS_g, SS_g;                         // gate/up stage strides (bytes)
    int WS_d, SS_d, d_row_copies;           // down stage strides, per-row copies (1) or one block copy (0)
    int use_push;
    PushCtx push;
    unsigned long long* trace;              // optional timeline [grid][kTraceEntries][4] (+ counts), see sl_moe_persist_trace
};

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(tc::smem_u32(dst)), "l"(src), "r"(bytes), "r"(tc::smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }
// Barrier of the consumer warps that also tells every one of them whether any saw `flag`: a wait that gave up makes all
// consumers leave together, so that none is left behind at a later barrier.
__device__ __forceinline__ bool consumer_any(bool flag) {
    uint32_t r;
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.u32 q, %1, 0;\n"
        "barrier.red.or.pred p, 1, %2, q;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(r) : "r"((uint32_t)flag), "n"(kConsumers) : "memory");
    return r != 0;
}

__device__ __forceinline__ void record_status(int* status, int site, int expected, int seen) {
    if (status != nullptr && atomicCAS(status, 0, 2) == 0) {
        status[1] = site;
        status[2] = expected;
        status[3] = seen;
    }
}

// Bounded mbarrier wait that also leaves when another thread of the block has given up.
__device__ __forceinline__ bool mbar_wait_abortable(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int site) {
    if (tc::mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = tc::globaltimer_ns();
    for (uint32_t i = 0;; ++i) {
        if (tc::mbar_try_wait(bar, parity)) return true;
        if ((i & 31u) == 31u) {
            if (*abort_flag) return false;
            if (tc::globaltimer_ns() - t0 > kWaitLimitNs) {
                record_status(status, site, (int)parity, -1);
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// Bounded wait until *counter >= target (acquire at GPU scope); one thread calls it.
__device__ __forceinline__ bool counter_wait(const uint32_t* counter, uint32_t target, volatile int* abort_flag, int* status, int site) {
    uint32_t seen = ld_acquire_gpu_u32(counter);
    if (seen >= target) return true;
    const uint64_t t0 = tc::globaltimer_ns();
    for (uint32_t i = 0;; ++i) {
        seen = ld_acquire_gpu_u32(counter);
        if (seen >= target) return true;
        if (*abort_flag) return false;
        if (i > 8) __nanosleep(i > 256 ? 200 : 40);
        if ((i & 63u) == 63u) {
            // another block already gave up: its tiles will never complete
            if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) { *abort_flag = 1; return false; }
            if (tc::globaltimer_ns() - t0 > kWaitLimitNs) {
                record_status(status, site, (int)target, (int)seen);
                *abort_flag = 1;
                return false;
            }
        }
    }
}

struct Smem {
    uint64_t stage_full[kStages], stage_empty[kStages], work_full[2], work_empty[2];
    Work work[2];
    int abort_flag;
    int wcnt[kConsumerWarps];
    int gates_done, downs_done;       // this block has seen every gate/up (down) tile of the layer completed
};

// ---- plan ---------------------------------------------------------------------------------------------------------
// Consumers only (256 threads, one routed route each).  Items 0 .. S-1 are the shared expert's chunks of eight tokens;
// routed items follow, numbered in the order of their first route, so the plan does not depend on thread timing.
__device__ void build_plan(const MoePersistParams& p, Smem* sm, const int* s_ids, int* base, int* table) {
    const int ctid = threadIdx.x - 32, lane = ctid & 31, cw = ctid >> 5;
    const int n = p.T * p.top_k, S = p.n_shared_items;
    for (int i = ctid; i < p.max_items * kItemRoutes; i += kConsumers) p.item_routes[i] = -1;
    for (int i = ctid; i < p.num_local; i += kConsumers) base[i] = 0;
    consumer_sync();
    int e = -1;
    if (ctid < n) {
        e = s_ids[ctid] - p.expert_offset;
        if (e < 0 || e >= p.num_local) e = -1;
    }
    const int key = e >= 0 ? e : -1 - lane;
    const unsigned mask = __match_any_sync(0xffffffffu, key);
    const int rank_w = __popc(mask & ((1u << lane) - 1u)), cnt_w = __popc(mask);
    int rank = 0;
    const int warps_used = (n + 31) / 32;
    for (int w = 0; w < warps_used; ++w) {
        if (cw == w) {
            if (e >= 0) rank = base[e] + rank_w;
            __syncwarp();
            if (e >= 0 && rank_w == 0) base[e] += cnt_w;
        }
        if (warps_used > 1) consumer_sync();
    }
    const int chunk = rank / kItemRoutes, within = rank % kItemRoutes;
    const bool lead = e >= 0 && within == 0;
    const unsigned lm = __ballot_sync(0xffffffffu, lead);
    if (lane == 0) sm->wcnt[cw] = __popc(lm);
    consumer_sync();
    int slot = S + __popc(lm & ((1u << lane) - 1u)), total = 0;
    for (int w = 0; w < kConsumerWarps; ++w) {
        if (w < cw) slot += sm->wcnt[w];
        total += sm->wcnt[w];
    }
    if (lead && slot < p.max_items) {
        table[e * 4 + chunk] = slot;
        p.item_expert[slot] = e;
    }
    consumer_sync();
    if (e >= 0) {
        const int s2 = table[e * 4 + chunk];
        if (s2 < p.max_items) p.item_routes[s2 * kItemRoutes + within] = ctid;
    }
    for (int i = ctid; i < S * kItemRoutes; i += kConsumers) {
        const int t = i;                      // shared route of token t lives in item t / 8, place t % 8
        if (t < p.T) p.item_routes[i] = n + t;
    }
    if (ctid < S) p.item_expert[ctid] = -1;
    if (ctid == 0) {
        const int items = S + total;
        *p.num_items = items < p.max_items ? items : p.max_items;
    }
}

template <int PER>
__device__ void route_tokens(const MoePersistParams& p, int* s_ids) {
    const int ctid = threadIdx.x - 32, lane = ctid & 31, cw = ctid >> 5;
    for (int t = cw; t < p.T; t += kConsumerWarps) {
        float lg[PER];
#pragma unroll
        for (int i = 0; i < PER; ++i) lg[i] = 0.f;
        for (int s = 0; s < p.RK; ++s) {
            const float* src = p.slabs + ((size_t)s * p.T + t) * p.E + lane * PER;
#pragma unroll
            for (int i = 0; i < PER; ++i)
                if (lane * PER + i < p.E) lg[i] += ldg_cg_f32(src + i);
        }
        int id; float w;
        route_warp<PER>(lg, p.bias, p.E, p.top_k, p.n_group, p.topk_group, p.norm, p.scale, id, w);
        if (lane < p.top_k) {
            p.ids[(size_t)t * p.top_k + lane] = id;
            p.wts[(size_t)t * p.top_k + lane] = w;
            s_ids[t * p.top_k + lane] = id;
        }
    }
}

// One block-wide completion signal: the barrier orders every consumer's stores before thread 0's fence, whose
// cumulativity publishes them at GPU scope before the counter moves.
__device__ __forceinline__ void signal_done(uint32_t* counter, uint32_t* counter2 = nullptr) {
    consumer_sync();
    if (threadIdx.x == 32) {
        __threadfence();
        atomicAdd(counter, 1u);
        if (counter2 != nullptr) atomicAdd(counter2, 1u);
    }
}

// ---- the kernel ---------------------------------------------------------------------------------------------------
template <int GPW>      // 128-index groups of H per consumer warp in a gate/up tile: H = 1024 * GPW
__global__ void __launch_bounds__(kThreads, 1) moe_persist_kernel(const __grid_constant__ MoePersistParams p) {
    pdl_grid_sync();
    extern __shared__ __align__(128) uint8_t dyn[];
    uint8_t* stages = dyn;
    uint8_t* xs = dyn + p.off_xs;                                  // T <= 8: the tokens' permuted f16 rows, padded
    float* scratch = reinterpret_cast<float*>(dyn + p.off_scratch);
    int* plan_sm = reinterpret_cast<int*>(dyn + p.off_plan);       // item_expert[max_items] | item_routes[max_items][8]
    Smem* sm = reinterpret_cast<Smem*>(dyn + p.off_ctl);
    volatile int* abort_flag = &sm->abort_flag;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_routed = p.T * p.top_k;
    const int NS = p.n_stages;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { tc::mbar_init(&sm->stage_full[s], 1); tc::mbar_init(&sm->stage_empty[s], kConsumerWarps); }
        for (int s = 0; s < 2; ++s) { tc::mbar_init(&sm->work_full[s], 1); tc::mbar_init(&sm->work_empty[s], kConsumerWarps); }
        sm->abort_flag = 0;
        sm->gates_done = 0;
        sm->downs_done = 0;
        tc::mbar_fence_init();
    }
    __syncthreads();

    if (warp == 0) {
        // ================================ producer ================================
        uint32_t it = 0;                       // stage uses issued so far
        int num_items = -1;
        const int n_shared_g = p.n_shared_items * p.TG;
        const int plan_idx = p.n_router + n_shared_g;
        int idx_next = 0;
        if (lane == 0) idx_next = (int)atomicAdd(&p.sync[kQueue], 1u);
        for (uint32_t wi = 0;; ++wi) {
            const int slot = wi & 1;
            int idx = __shfl_sync(0xffffffffu, idx_next, 0);
            bool ok = true;
            if (idx > plan_idx && num_items < 0) {
                // first tile behind the plan: wait for it once and keep a copy of the plan in shared memory
                if (lane == 0) ok = counter_wait(&p.sync[kPlanDone], 1u, abort_flag, p.status, 1);
                ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
                if (!ok) break;
                num_items = ldg_cg_i32(p.num_items);
                for (int i = lane; i < num_items; i += 32) plan_sm[i] = ldg_cg_i32(p.item_expert + i);
                for (int i = lane; i < num_items * kItemRoutes; i += 32) plan_sm[p.max_items + i] = ldg_cg_i32(p.item_routes + i);
                __syncwarp();
            }
            // the claim of the next tile travels while this one is set up and its weights are requested
            if (lane == 0) idx_next = (int)atomicAdd(&p.sync[kQueue], 1u);
            int kind = kExit, item = 0, blk = 0, ex = 0, route = -1;         // `route`: lane q < 8 holds the item's q-th route
            if (idx < p.n_router) {
                kind = kRouter; item = idx / p.RK; blk = idx % p.RK;
            } else if (idx < plan_idx) {
                idx -= p.n_router;
                kind = kGate; item = idx / p.TG; blk = idx % p.TG; ex = -1;
                const int t = item * kItemRoutes + lane;
                route = (lane < kItemRoutes && t < p.T) ? n_routed + t : -1;
            } else if (idx == plan_idx) {
                kind = kPlan;
            } else {
                idx -= plan_idx + 1;
                const int nri = num_items - p.n_shared_items;
                if (idx < nri * p.TG) {
                    kind = kGate; item = p.n_shared_items + idx / p.TG; blk = idx % p.TG;
                } else if (idx < nri * p.TG + num_items * p.TD) {
                    idx -= nri * p.TG;
                    kind = kDown; item = idx / p.TD; blk = idx % p.TD;
                } else if (idx < nri * p.TG + num_items * p.TD + p.T * p.NXB) {
                    idx -= nri * p.TG + num_items * p.TD;
                    kind = kReduce; item = idx / p.NXB; blk = idx % p.NXB;
                }
                if (kind == kGate || kind == kDown) {
                    ex = plan_sm[item];
                    if (lane < kItemRoutes) route = plan_sm[p.max_items + item * kItemRoutes + lane];
                }
            }
            if (lane == 0) ok = mbar_wait_abortable(&sm->work_empty[slot], ((wi >> 1) & 1u) ^ 1u, abort_flag, p.status, 2);
            ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
            if (!ok) break;
            if (lane < kItemRoutes) sm->work[slot].routes[lane] = route;
            if (lane == 0) { sm->work[slot].kind = kind; sm->work[slot].item = item; sm->work[slot].expert = ex; sm->work[slot].blk = blk; }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&sm->work_full[slot]);
            if (kind == kExit) break;
            // ---- weight streaming ----
            int n_sub = 0;
            if (kind == kRouter) n_sub = 1;
            else if (kind == kGate) n_sub = p.gsub;
            else if (kind == kDown) n_sub = p.dsub;
            for (int s = 0; s < n_sub && ok; ++s, ++it) {
                const int st = it % NS;
                uint8_t* dst = stages + (size_t)st * kStageBytes;
                uint64_t* full = &sm->stage_full[st];
                if (lane == 0) ok = mbar_wait_abortable(&sm->stage_empty[st], ((it / NS) & 1u) ^ 1u, abort_flag, p.status, 3);
                ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
                if (!ok) break;
                if (kind == kRouter) {
                    const uint32_t rb = (uint32_t)p.KC * 2u;
                    if (lane == 0) tc::mbar_expect_tx(full, 16u * rb);
                    __syncwarp();
                    if (lane < 16)
                        bulk_g2s(dst + (size_t)lane * (rb + 16), p.router_w + (size_t)(item * 16 + lane) * p.H + (size_t)blk * p.KC, rb, full);
                } else if (kind == kGate) {
                    const uint8_t* W = ex < 0 ? p.sw13 : p.w13 + (size_t)ex * 2 * p.I * (p.H / 2);
                    const uint8_t* S = ex < 0 ? p.ss13 : p.s13 + (size_t)ex * 2 * p.I * (p.H / 16);
                    const int i0 = (blk * p.gsub + s) * 8;
                    const uint32_t wb = (uint32_t)p.H / 2, sb = (uint32_t)p.H / 16;
                    if (lane == 0) tc::mbar_expect_tx(full, 16u * (wb + sb));
                    __syncwarp();
                    const int r = lane & 15;
                    const int grow = r < 8 ? i0 + r : p.I + i0 + (r - 8);       // gate rows, then up rows
                    if (lane < 16) bulk_g2s(dst + (size_t)r * p.WS_g, W + (size_t)grow * wb, wb, full);
                    else bulk_g2s(dst + (size_t)16 * p.WS_g + (size_t)r * p.SS_g, S + (size_t)grow * sb, sb, full);
                } else {
                    const uint8_t* W = ex < 0 ? p.sw2 : p.w2 + (size_t)ex * p.H * (p.I / 2);
                    const uint8_t* S = ex < 0 ? p.ss2 : p.s2 + (size_t)ex * p.H * (p.I / 16);
                    const int rows = p.drep * p.RTd * 16;
                    const int n0 = (blk * p.dsub + s) * rows;
                    const uint32_t wb = (uint32_t)p.I / 2, sb = (uint32_t)p.I / 16;
                    if (lane == 0) tc::mbar_expect_tx(full, (uint32_t)rows * (wb + sb));
                    __syncwarp();
                    if (p.d_row_copies) {
                        for (int r = lane; r < rows; r += 32) {
                            bulk_g2s(dst + (size_t)r * p.WS_d, W + (size_t)(n0 + r) * wb, wb, full);
                            bulk_g2s(dst + (size_t)rows * p.WS_d + (size_t)r * p.SS_d, S + (size_t)(n0 + r) * sb, sb, full);
                        }
                    } else if (lane == 0) {
                        bulk_g2s(dst, W + (size_t)n0 * wb, (uint32_t)rows * wb, full);
                        bulk_g2s(dst + (size_t)rows * p.WS_d, S + (size_t)n0 * sb, (uint32_t)rows * sb, full);
                    }
                }
            }
            if (!ok) break;
        }
        // leave no copy in flight behind: the last uses of every stage have either been consumed or complete here
        if (lane == 0 && *abort_flag) {
            const uint32_t lo = it > (uint32_t)NS ? it - NS : 0u;
            for (uint32_t k = lo; k < it; ++k) tc::mbar_wait(&sm->stage_full[k % NS], (k / NS) & 1u, 2000000ull);
        }
    } else {
        // ================================ consumers ================================
        const int ctid = tid - 32, cw = warp - 1;
        const int g = lane >> 2, c = lane & 3;
        const int G = p.H / 128;
        const int xs_stride = G * 256 + 64;                      // bytes per token row of `xs`
        bool xs_ready = false;
        uint32_t it = 0;
        for (uint32_t wi = 0;; ++wi) {
            const int slot = wi & 1;
            if (consumer_any(!mbar_wait_abortable(&sm->work_full[slot], (wi >> 1) & 1u, abort_flag, p.status, 4))) break;
            const int kind = sm->work[slot].kind, item = sm->work[slot].item, expert = sm->work[slot].expert, blk = sm->work[slot].blk;
            const int route_g = sm->work[slot].routes[g];                     // the route in MMA column g
            const int route_e = sm->work[slot].routes[(ctid >> 4) & 7];       // the route this thread finishes in the epilogues
            const int route_e8 = sm->work[slot].routes[(ctid >> 3) & 7];
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&sm->work_empty[slot]);
            if (kind == kExit) break;
            bool ok = true;
            unsigned long long t_start = 0, t_ready = 0, t_mid = 0;
            if (p.trace != nullptr && ctid == 0) t_start = tc::globaltimer_ns();

            if (kind == kRouter) {
                // ---- 16 router rows x K chunk, all tokens: bf16 tensor cores, k16 steps dealt round-robin to the warps ----
                const int st = it % NS;
                const int NT = (p.T + 7) / 8;
                const int steps = p.KC / 16;
                // one token tile: this warp's activation fragments are loaded before the weights arrive
                uint32_t xb[12][2];
                if (NT == 1) {
#pragma unroll
                    for (int q = 0; q < 12; ++q) {
                        const int ks = cw + q * kConsumerWarps;
                        xb[q][0] = xb[q][1] = 0u;
                        if (ks < steps && g < p.T) {
                            const bf16* xr = p.x + (size_t)g * p.ldx + (size_t)blk * p.KC + ks * 16 + 2 * c;
                            xb[q][0] = *reinterpret_cast<const uint32_t*>(xr);
                            xb[q][1] = *reinterpret_cast<const uint32_t*>(xr + 8);
                        }
                    }
                }
                ok = mbar_wait_abortable(&sm->stage_full[st], (it / NS) & 1u, abort_flag, p.status, 5);
                if (consumer_any(!ok)) break;
                if (p.trace != nullptr && ctid == 0) t_ready = tc::globaltimer_ns();
                const uint8_t* Wsm = stages + (size_t)st * kStageBytes;
                const int WSr = p.KC * 2 + 16;
                float acc[4][4];
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
                for (int q = 0; q < 12; ++q) {
                    const int ks = cw + q * kConsumerWarps;
                    if (ks < steps) {
                        const int k0 = ks * 16;
                        uint32_t a[4];
                        a[0] = *reinterpret_cast<const uint32_t*>(Wsm + (size_t)g * WSr + (k0 + 2 * c) * 2);
                        a[1] = *reinterpret_cast<const uint32_t*>(Wsm + (size_t)(g + 8) * WSr + (k0 + 2 * c) * 2);
                        a[2] = *reinterpret_cast<const uint32_t*>(Wsm + (size_t)g * WSr + (k0 + 8 + 2 * c) * 2);
                        a[3] = *reinterpret_cast<const uint32_t*>(Wsm + (size_t)(g + 8) * WSr + (k0 + 8 + 2 * c) * 2);
                        if (NT == 1) {
                            mma_bf16_m16n8k16(acc[0], a, xb[q][0], xb[q][1]);
                        } else {
#pragma unroll
                            for (int nt = 0; nt < 4; ++nt) {
                                if (nt < NT) {
                                    const int tok = nt * 8 + g;
                                    uint32_t b0 = 0, b1 = 0;
                                    if (tok < p.T) {
                                        const bf16* xr = p.x + (size_t)tok * p.ldx + (size_t)blk * p.KC + k0 + 2 * c;
                                        b0 = *reinterpret_cast<const uint32_t*>(xr);
                                        b1 = *reinterpret_cast<const uint32_t*>(xr + 8);
                                    }
                                    mma_bf16_m16n8k16(acc[nt], a, b0, b1);
                                }
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&sm->stage_empty[st]);
                ++it;
                float* mine = scratch + (size_t)cw * (NT * 128);
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    if (nt < NT) {
                        mine[nt * 128 + (2 * c) * 16 + g] = acc[nt][0];
                        mine[nt * 128 + (2 * c + 1) * 16 + g] = acc[nt][1];
                        mine[nt * 128 + (2 * c) * 16 + g + 8] = acc[nt][2];
                        mine[nt * 128 + (2 * c + 1) * 16 + g + 8] = acc[nt][3];
                    }
                }
                consumer_sync();
                for (int i = ctid; i < NT * 128; i += kConsumers) {
                    const int tok = i >> 4, r = i & 15;
                    if (tok < p.T) {
                        float v = 0.f;
                        for (int w = 0; w < kConsumerWarps; ++w) v += scratch[(size_t)w * (NT * 128) + i];
                        p.slabs[((size_t)blk * p.T + tok) * p.E + item * 16 + r] = v;
                    }
                }
                signal_done(&p.sync[kRouterDone]);

            } else if (kind == kPlan) {
                int* s_ids = reinterpret_cast<int*>(scratch);          // [256]
                int* base = s_ids + 256;                                // [num_local]
                int* table = base + p.num_local;                        // [num_local * 4]
                if (p.router_w != nullptr) {
                    if (ctid == 0) ok = counter_wait(&p.sync[kRouterDone], (uint32_t)p.n_router, abort_flag, p.status, 6);
                    if (consumer_any(!ok)) break;
                    if (p.trace != nullptr && ctid == 0) t_ready = tc::globaltimer_ns();
                    int PER = 1;
                    while (PER * 32 < p.E) PER <<= 1;
                    switch (PER) {
                        case 1: route_tokens<1>(p, s_ids); break;
                        case 2: route_tokens<2>(p, s_ids); break;
                        case 4: route_tokens<4>(p, s_ids); break;
                        case 8: route_tokens<8>(p, s_ids); break;
                        default: route_tokens<16>(p, s_ids); break;
                    }
                } else {
                    for (int i = ctid; i < n_routed; i += kConsumers) s_ids[i] = p.ids[i];
                }
                consumer_sync();
                if (p.trace != nullptr && ctid == 0) t_mid = tc::globaltimer_ns();
                build_plan(p, sm, s_ids, base, table);
                consumer_sync();
                if (ctid == 0) {
                    __threadfence();
                    atomicExch(&p.sync[kPlanDone], 1u);
                }

            } else if (kind == kGate) {
                // ---- activations of the item's routes: this warp's groups of every sub-tile ----
                // T <= 8: MMA column g is token g for every item (the tokens' rows sit in shared memory once per block);
                // more tokens: column g is the item's g-th route and its token's row comes from global memory.
                if (p.xs_mode && !xs_ready) {
                    const int units = 8 * G * 16;
                    for (int u = ctid; u < units; u += kConsumers) {
                        const int tok = u / (G * 16), rest = u % (G * 16);
                        *reinterpret_cast<uint4*>(xs + (size_t)tok * xs_stride + (size_t)rest * 16) = ldg_ca_16(p.xp + u);
                    }
                    xs_ready = true;
                    consumer_sync();
                }
                uint4 xv[GPW][4];
                if (p.xs_mode) {
#pragma unroll
                    for (int gi = 0; gi < GPW; ++gi) {
                        const uint8_t* xr = xs + (size_t)g * xs_stride + (size_t)((cw + kConsumerWarps * gi) * 16 + c) * 16;
#pragma unroll
                        for (int j = 0; j < 4; ++j) xv[gi][j] = *reinterpret_cast<const uint4*>(xr + j * 64);
                    }
                } else {
                    const int tok = route_g < 0 ? 0 : (route_g < n_routed ? route_g / p.top_k : route_g - n_routed);
#pragma unroll
                    for (int gi = 0; gi < GPW; ++gi) {
                        const uint4* xr = p.xp + ((size_t)tok * G + (cw + kConsumerWarps * gi)) * 16 + c;
#pragma unroll
                        for (int j = 0; j < 4; ++j) xv[gi][j] = ldg_ca_16(xr + j * 4);
                    }
                }
                if (p.trace != nullptr && ctid == 0) t_ready = tc::globaltimer_ns();
                const float* Gs = expert < 0 ? p.sg13 : p.g13 + (size_t)expert * 2;
                const float gg = Gs[0], gu = Gs[1];
                const int Gd = p.I / 128;
                // epilogue role of threads 0..63: route place (ctid >> 3), gate/up column pair (ctid & 7)
                const int ecol = route_e8 < 0 ? 0 : (p.xs_mode ? (route_e8 < n_routed ? route_e8 / p.top_k : route_e8 - n_routed) : ((ctid >> 3) & 7));
                __half* act = reinterpret_cast<__half*>(p.act_perm);
                for (int s = 0; s < p.gsub; ++s, ++it) {
                    const int st = it % NS;
                    ok = !consumer_any(!mbar_wait_abortable(&sm->stage_full[st], (it / NS) & 1u, abort_flag, p.status, 7));
                    if (!ok) break;
                    const uint8_t* Wsm = stages + (size_t)st * kStageBytes;
                    const uint8_t* Ssm = Wsm + (size_t)16 * p.WS_g;
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int gi = 0; gi < GPW; ++gi) {
                        const int group = cw + kConsumerWarps * gi;
                        const int kk = group * 128 + c * 32;
                        const uint4 w0 = *reinterpret_cast<const uint4*>(Wsm + (size_t)g * p.WS_g + (kk >> 1));
                        const uint4 w1 = *reinterpret_cast<const uint4*>(Wsm + (size_t)(g + 8) * p.WS_g + (kk >> 1));
                        const uint16_t s0 = *reinterpret_cast<const uint16_t*>(Ssm + (size_t)g * p.SS_g + (kk >> 4));
                        const uint16_t s1 = *reinterpret_cast<const uint16_t*>(Ssm + (size_t)(g + 8) * p.SS_g + (kk >> 4));
                        __half2 lo[16], hi[16];
                        expand_row(w0, s0, lo);
                        expand_row(w1, s1, hi);
                        mma_group_w4(acc, lo, hi, xv[gi]);
                    }
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(&sm->stage_empty[st]);
                    // rows 0..7 = gate columns i0..i0+7, rows 8..15 = the matching up columns
                    float* mine = scratch + (size_t)cw * 128;
                    mine[(2 * c) * 16 + g] = acc[0];
                    mine[(2 * c + 1) * 16 + g] = acc[1];
                    mine[(2 * c) * 16 + g + 8] = acc[2];
                    mine[(2 * c + 1) * 16 + g + 8] = acc[3];
                    consumer_sync();
                    if (ctid < 64 && route_e8 >= 0) {
                        const int pcol = ctid & 7;
                        float gs = 0.f, us = 0.f;
                        for (int w = 0; w < kConsumerWarps; ++w) {
                            gs += scratch[(size_t)w * 128 + ecol * 16 + pcol];
                            us += scratch[(size_t)w * 128 + ecol * 16 + 8 + pcol];
                        }
                        gs *= gg; us *= gu;
                        const float a = gs / (1.f + __expf(-gs)) * us;
                        const int i = (blk * p.gsub + s) * 8 + pcol;
                        const int w128 = i % 128, cc = w128 / 32, jj = (w128 % 32) / 8, ee = w128 % 8;
                        act[((((size_t)route_e8 * Gd + i / 128) * 16 + jj * 4 + cc) * 8) + ee] = __float2half(a);
                    }
                    consumer_sync();
                }
                if (!ok) break;
                signal_done(&p.sync[kGateDone + item], &p.sync[kGateTotal]);

            } else if (kind == kDown) {
                if (ctid == 0 && !sm->gates_done) {
                    ok = counter_wait(&p.sync[kGateDone + item], (uint32_t)p.TG, abort_flag, p.status, 8);
                    // once every gate/up tile of the layer is complete, later down tiles of this block skip the wait
                    if (ok && ld_acquire_gpu_u32(&p.sync[kGateTotal]) >= (uint32_t)(ldg_cg_i32(p.num_items) * p.TG)) sm->gates_done = 1;
                }
                if (consumer_any(!ok)) break;
                if (p.trace != nullptr && ctid == 0) t_ready = tc::globaltimer_ns();
                const int GI = p.I / 128;
                const int rt = cw / p.KSd, kp = cw % p.KSd;
                const int gpw = GI / p.KSd;                              // 1 or 2
                uint4 av[2][4];
#pragma unroll
                for (int gi = 0; gi < 2; ++gi) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) av[gi][j] = make_uint4(0, 0, 0, 0);
                    if (gi < gpw && route_g >= 0) {
                        const uint4* ar = p.act_perm + ((size_t)route_g * GI + (kp + p.KSd * gi)) * 16 + c;
#pragma unroll
                        for (int j = 0; j < 4; ++j) av[gi][j] = ldg_cg_16(ar + j * 4);
                    }
                }
                const float gs2 = expert < 0 ? p.sg2[0] : p.g2[expert];
                const int rep_rows = p.RTd * 16, rows = p.drep * rep_rows;
                for (int s = 0; s < p.dsub; ++s, ++it) {
                    const int st = it % NS;
                    ok = !consumer_any(!mbar_wait_abortable(&sm->stage_full[st], (it / NS) & 1u, abort_flag, p.status, 9));
                    if (!ok) break;
                    const uint8_t* Wsm = stages + (size_t)st * kStageBytes;
                    const uint8_t* Ssm = Wsm + (size_t)rows * p.WS_d;
                    const int n0 = (blk * p.dsub + s) * rows;
                    for (int rep = 0; rep < p.drep; ++rep) {
                        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int gi = 0; gi < 2; ++gi) {
                            if (gi < gpw) {
                                const int group = kp + p.KSd * gi;
                                const int kk = group * 128 + c * 32;
                                const int ra = rep * rep_rows + rt * 16 + g, rb = ra + 8;
                                const uint4 w0 = *reinterpret_cast<const uint4*>(Wsm + (size_t)ra * p.WS_d + (kk >> 1));
                                const uint4 w1 = *reinterpret_cast<const uint4*>(Wsm + (size_t)rb * p.WS_d + (kk >> 1));
                                const uint16_t s0 = *reinterpret_cast<const uint16_t*>(Ssm + (size_t)ra * p.SS_d + (kk >> 4));
                                const uint16_t s1 = *reinterpret_cast<const uint16_t*>(Ssm + (size_t)rb * p.SS_d + (kk >> 4));
                                __half2 lo[16], hi[16];
                                expand_row(w0, s0, lo);
                                expand_row(w1, s1, hi);
                                mma_group_w4(acc, lo, hi, av[gi]);
                            }
                        }
                        if (rep == p.drep - 1) {
                            __syncwarp();
                            if (lane == 0) tc::mbar_arrive(&sm->stage_empty[st]);
                        }
                        float* mine = scratch + (size_t)cw * 128;
                        mine[(2 * c) * 16 + g] = acc[0];
                        mine[(2 * c + 1) * 16 + g] = acc[1];
                        mine[(2 * c) * 16 + g + 8] = acc[2];
                        mine[(2 * c + 1) * 16 + g + 8] = acc[3];
                        consumer_sync();
                        if (route_e >= 0) {
                            for (int i = ctid; i < p.RTd * 128; i += kConsumers) {
                                const int t2 = i >> 7, rem = i & 127, r = rem & 15;
                                float v = 0.f;
                                for (int k2 = 0; k2 < p.KSd; ++k2) v += scratch[(size_t)(t2 * p.KSd + k2) * 128 + rem];
                                p.y_route[(size_t)route_e * p.H + n0 + rep * rep_rows + t2 * 16 + r] = v * gs2;
                            }
                        }
                        consumer_sync();
                    }
                }
                if (!ok) break;
                signal_done(&p.sync[kDownDone]);

            } else {   // kReduce: out[t, n] = sum_j wt[t, j] * y_route[t * k + j, n] (local experts) + y_route[shared(t), n]
                if (ctid == 0 && !sm->downs_done) {
                    ok = counter_wait(&p.sync[kDownDone], (uint32_t)(ldg_cg_i32(p.num_items) * p.TD), abort_flag, p.status, 10);
                    if (ok) sm->downs_done = 1;
                }
                if (consumer_any(!ok)) break;
                if (p.trace != nullptr && ctid == 0) t_ready = tc::globaltimer_ns();
                const int t = item, n = blk * 1024 + ctid * 4;
                if (n < p.H) {
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int j = 0; j < p.top_k; ++j) {
                        const int e = ldg_cg_i32(p.ids + t * p.top_k + j) - p.expert_offset;
                        if (e >= 0 && e < p.num_local) {
                            const float w = ldg_cg_f32(p.wts + t * p.top_k + j);
                            const uint4 u = ldg_cg_16(p.y_route + (size_t)(t * p.top_k + j) * p.H + n);
                            v.x += w * __uint_as_float(u.x); v.y += w * __uint_as_float(u.y);
                            v.z += w * __uint_as_float(u.z); v.w += w * __uint_as_float(u.w);
                        }
                    }
                    if (p.n_shared_items > 0) {
                        const uint4 u = ldg_cg_16(p.y_route + (size_t)(n_routed + t) * p.H + n);
                        v.x += __uint_as_float(u.x); v.y += __uint_as_float(u.y); v.z += __uint_as_float(u.z); v.w += __uint_as_float(u.w);
                    }
                    if (p.use_push) {
                        const uint32_t ptag = push_tag(p.push);
                        push_store_all(p.push, t, n, v.x, ptag);
                        push_store_all(p.push, t, n + 1, v.y, ptag);
                        push_store_all(p.push, t, n + 2, v.z, ptag);
                        push_store_all(p.push, t, n + 3, v.w, ptag);
                    } else {
                        *reinterpret_cast<float4*>(p.out + (size_t)t * p.H + n) = v;
                    }
                }
            }
            if (p.trace != nullptr && ctid == 0 && wi < (uint32_t)kTraceEntries) {
                unsigned long long* e = p.trace + ((size_t)blockIdx.x * kTraceEntries + wi) * 4;
                e[0] = ((unsigned long long)kind << 32) | ((unsigned long long)(item & 0xffff) << 8) | (unsigned)(blk & 0xff);
                e[1] = t_start; e[2] = t_ready; e[3] = tc::globaltimer_ns();
                if (kind == kPlan) {                  // the plan tile's halves: routing done, plan built
                    unsigned long long* e2 = p.trace + ((size_t)blockIdx.x * kTraceEntries + kTraceEntries - 1) * 4;
                    e2[0] = 99ull << 32; e2[1] = t_ready; e2[2] = t_mid; e2[3] = e[3];
                }
            }
        }
    }
    __syncthreads();
    // the block that leaves last puts the counters back to zero for the next launch (not after a failed wait:
    // the host clears them when it reads the status)
    if (tid == 0 && !*abort_flag) {
        __threadfence();
        const uint32_t ticket = atomicAdd(&p.sync[kExitCount], 1u);
        if (ticket == gridDim.x - 1) {
            for (int i = 0; i < kGateDone + p.max_items; ++i) p.sync[i] = 0u;
            __threadfence();
        }
    }
}

struct DeviceInfo { int sms; };
DeviceInfo device_info() {
    static int sms[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return {148};
    if (sms[dev] == 0) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    return {sms[dev] > 0 ? sms[dev] : 148};
}

int round_up(int v, int m) { return (v + m - 1) / m * m; }

}  // namespace

struct MoePersistArgs {
    const void* x; int ldx;
    const void* xp;
    const void* router_w; const void* bias;
    int E, n_group, topk_group, norm;
    float scale;
    int T, top_k, H, I, expert_offset, num_local;
    const void *w13, *s13, *g13, *sw13, *ss13, *sg13;
    const void *w2, *s2, *g2, *sw2, *ss2, *sg2;
    void* slabs;          // f32 [4][T][E]
    void* act_perm;       // f16 [routes + 8][I]
    void* y_route;        // f32 [routes][H]
    void* plan;           // int32 [max_items * 9 + 1]
    void* ids; void* wts; // [T, top_k]: outputs with a router stage, inputs without
    void* sync;           // u32 [8 + max_items], zero before the first launch; the kernel leaves it zero
    void* status;         // int32 [4]
    void* out;            // f32 [T, H] (ignored when pushing)
    int max_items;        // >= ceil(T/8) (shared) + T * top_k
    int gsub;             // gate/up sub-tiles per tile (0 = default)
    void* trace;          // optional u64 [grid][96][4] timeline of the tiles each block worked on (zeroed by the caller), or null
};

// Shapes the persistent kernel takes; everything else stays on the five-launch path.
SL_API int sl_moe_persist_ok(int T, int top_k, int H, int I, int E, int num_local, int has_router) {
    if (T < 1 || T > 32 || T * top_k > 256 || top_k > 32) return 0;
    if (H % 1024 != 0 || H / 1024 > 6 || H / 1024 == 5) return 0;
    const int GI = I / 128;
    if (I % 128 != 0 || !(GI == 1 || GI == 2 || GI == 4 || GI == 8 || GI == 16)) return 0;
    if (num_local > 512) return 0;
    if (has_router && (E % 16 != 0 || E > 512)) return 0;
    if (16 * (round_up(H / 2, 128) + 64 + round_up(H / 16, 128) + 16) > kStageBytes) return 0;
    return 1;
}

SL_API int sl_moe_persist(const MoePersistArgs* a, const PushCtx* push, cudaStream_t s) {
    if (a->T == 0) return 0;
    const int has_router = a->router_w != nullptr;
    if (!sl_moe_persist_ok(a->T, a->top_k, a->H, a->I, a->E, a->num_local, has_router)) return -1;
    if (push != nullptr && (a->T > push->slot_rows || a->H > push->row_len)) return -1;
    if (has_router) {
        if (a->n_group < 1 || a->n_group > 32 || a->E % a->n_group != 0) return -1;
        int PER = 1;
        while (PER * 32 < a->E) PER <<= 1;
        if (a->n_group > 1) {
            const int gsz = a->E / a->n_group;
            if (gsz % PER != 0) return -1;
            const int lpg = gsz / PER;
            if (lpg & (lpg - 1)) return -1;
        }
    }
    const int has_shared = a->sw13 != nullptr;
    MoePersistParams p{};
    p.x = (const bf16*)a->x; p.ldx = a->ldx; p.xp = (const uint4*)a->xp;
    p.router_w = (const bf16*)a->router_w; p.bias = (const float*)a->bias;
    p.E = a->E; p.n_group = a->n_group; p.topk_group = a->topk_group; p.norm = a->norm; p.scale = a->scale;
    p.T = a->T; p.top_k = a->top_k; p.H = a->H; p.I = a->I; p.expert_offset = a->expert_offset; p.num_local = a->num_local;
    p.w13 = (const uint8_t*)a->w13; p.s13 = (const uint8_t*)a->s13; p.g13 = (const float*)a->g13;
    p.sw13 = (const uint8_t*)a->sw13; p.ss13 = (const uint8_t*)a->ss13; p.sg13 = (const float*)a->sg13;
    p.w2 = (const uint8_t*)a->w2; p.s2 = (const uint8_t*)a->s2; p.g2 = (const float*)a->g2;
    p.sw2 = (const uint8_t*)a->sw2; p.ss2 = (const uint8_t*)a->ss2; p.sg2 = (const float*)a->sg2;
    p.slabs = (float*)a->slabs; p.act_perm = (uint4*)a->act_perm; p.y_route = (float*)a->y_route;
    int* plan = (int*)a->plan;
    p.item_expert = plan; p.item_routes = plan + a->max_items; p.num_items = plan + a->max_items * (1 + kItemRoutes);
    p.ids = (int*)a->ids; p.wts = (float*)a->wts;
    p.sync = (uint32_t*)a->sync; p.status = (int*)a->status; p.out = (float*)a->out; p.max_items = a->max_items;
    p.n_shared_items = has_shared ? (a->T + 7) / 8 : 0;
    if (a->max_items < p.n_shared_items + a->T * a->top_k) return -1;
    // router: 16 rows x KC per tile, KC the largest divisor of H (a multiple of 128) whose tile fits a stage
    p.RK = 1;
    while (16 * ((a->H / p.RK) * 2 + 16) > kStageBytes || a->H % (p.RK * 128) != 0) {
        if (++p.RK > 4) return -1;
    }
    p.KC = a->H / p.RK;
    p.n_router = has_router ? (a->E / 16) * p.RK : 0;
    const int G = a->H / 128;
    // T <= 8: the tokens' permuted rows stay in shared memory for the whole kernel (two weight stages instead of three)
    const int NT = (a->T + 7) / 8;
    const int xs_bytes = 8 * (G * 256 + 64);
    int scratch_bytes = kConsumerWarps * NT * 128 * (int)sizeof(float);
    const int plan_scratch = (256 + 5 * a->num_local) * (int)sizeof(int);
    if (plan_scratch > scratch_bytes) scratch_bytes = plan_scratch;
    scratch_bytes = round_up(scratch_bytes, 128);
    const int plan_bytes = round_up(a->max_items * (1 + kItemRoutes) * (int)sizeof(int), 128);
    const int ctl_bytes = round_up((int)sizeof(Smem), 128);
    p.xs_mode = a->T <= 8 && 2 * kStageBytes + xs_bytes + scratch_bytes + plan_bytes + ctl_bytes <= 227 * 1024;
    p.n_stages = p.xs_mode ? 2 : kStages;
    p.off_xs = p.n_stages * kStageBytes;
    p.off_scratch = p.off_xs + (p.xs_mode ? xs_bytes : 0);
    p.off_plan = p.off_scratch + scratch_bytes;
    p.off_ctl = p.off_plan + plan_bytes;
    const size_t smem = (size_t)p.off_ctl + ctl_bytes;
    if (smem > 227 * 1024) return -1;
    // gate/up: with resident tokens a tile costs nothing to set up, so tiles stay small (better balance); otherwise four
    // sub-tiles share one load of the item's token rows
    p.gsub = a->gsub > 0 ? a->gsub : (p.xs_mode ? 2 : 4);
    while ((a->I / 8) % p.gsub != 0) --p.gsub;
    p.TG = a->I / (8 * p.gsub);
    const int GI = a->I / 128;
    p.KSd = GI >= 2 ? GI / 2 : 1;
    p.RTd = kConsumerWarps / p.KSd;
    p.d_row_copies = (a->I / 2) >= 512 ? 1 : 0;
    if (p.d_row_copies) {
        p.WS_d = round_up(a->I / 2, 128) + 64;
        p.SS_d = round_up(a->I / 16, 128) + 16;
    } else {
        p.WS_d = a->I / 2;
        p.SS_d = a->I / 16;
    }
    // down: a sub-tile holds `drep` passes of RTd * 16 rows (as many as fit a stage), a tile `dsub` sub-tiles
    const int pass_bytes = p.RTd * 16 * (p.WS_d + p.SS_d);
    if (pass_bytes > kStageBytes) return -1;
    p.drep = kStageBytes / pass_bytes;
    if (p.drep > 4) p.drep = 4;
    while (a->H % (p.drep * p.RTd * 16) != 0) --p.drep;
    p.dsub = 2;
    while (a->H % (p.dsub * p.drep * p.RTd * 16) != 0) --p.dsub;
    p.TD = a->H / (p.dsub * p.drep * p.RTd * 16);
    p.NXB = (a->H + 1023) / 1024;
    p.WS_g = round_up(a->H / 2, 128) + 64;
    p.SS_g = round_up(a->H / 16, 128) + 16;
    p.trace = (unsigned long long*)a->trace;
    p.use_push = push != nullptr;
    if (push != nullptr) p.push = *push;

    const int grid = device_info().sms;
    auto launch = [&](auto kern) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        sl_launch(kern, grid, kThreads, smem, s, p);
    };
    switch (a->H / 1024) {
        case 1: launch(moe_persist_kernel<1>); break;
        case 2: launch(moe_persist_kernel<2>); break;
        case 3: launch(moe_persist_kernel<3>); break;
        case 4: launch(moe_persist_kernel<4>); break;
        default: launch(moe_persist_kernel<6>); break;
    }
    return (int)cudaGetLastError();
}
