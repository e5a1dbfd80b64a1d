// Sparse MLA attention (prefill and decode) on the 5th-generation tensor cores, straight from the FP8 cache rows.
//
//   o[t, h, :] = sum_j softmax_j(q[t, h] . k[j]) v[j]     j over the token's selected rows (top-k), 8 heads per CTA
//
// A cache row is 656 bytes: 512 e4m3 latent codes, four fp32 scales (one per 128 codes), 64 bf16 rope values.  The
// mma.sync kernels spend their issue slots expanding those codes to f16 in shared memory; here the codes are never
// expanded.  One CTA works on one (query token, group of 8 heads, key split) at a time and walks that split's rows in
// tiles of 128 keys.  With one split (prefill) the item writes the final bf16 rows; with several (decode: one tile per
// split) its normalised fp32 partial and log-sum-exp, which the merge kernel combines (`csrc/sparse_mla.cu`).
//
//   gather   `cp.async` (16 bytes, zero fill for rows past the token's length) copies each row's four 128-byte code
//            groups into four K-major 128-byte-swizzled tiles [128 keys x 128 bytes], the rope part into a fifth
//            tile and the scales aside.  A warp copies whole rows (lane = 16-byte piece).  A CTA holds one key tile
//            and runs its phases one after the other; two CTAs share an SM (2 x 110 KB of shared memory, 2 x 256
//            TMEM columns, 2 x 256 threads with the whole register file), so one gathers while the other computes.
//   S^T      keys on the 128 MMA rows, N = 16 columns: `kind::f8f6f4` needs both operands in 8 bits, so the query is
//            split into two e4m3 terms (q * 2^e = hi + lo / 16; columns h and 8 + h) with a per-head power-of-two
//            scale.  One accumulator per code group (the key's group scale is applied to the group sums by the thread
//            that owns the key's TMEM lane) and one `kind::f16` accumulator for the rope part: 5 x 16 columns.
//   softmax  two threads own key j (four heads each): s = sum_g scale[g] (hi_g + lo_g / 16) / 2^e + rope, in log2
//            units.  The running maximum is a reference that is only raised when a value exceeds it by more than 2^8, and then to 2^6 below
//            the largest value seen; exponentials are taken relative to it (at most 2^8, and resolved down to 2^-19 of the
//            row maximum by the two e4m3 terms).  The value scale is folded into P (P_g = p * scale[g]); to keep P_g inside the
//            e4m3 range whatever the scales are, the reference tracks s + log2(max_g scale[g]).  P_g is again two
//            e4m3 terms and is written as the K-major B operand [16 columns x 128 keys] of the second product.
//   O^T      the same code tiles read MN-major (128 latent dims of a group on the MMA rows, keys on K): four
//            accumulators [128 dims x 16 columns] that stay in TMEM across tiles.  When the reference is raised the
//            accumulators are folded into registers with the correction factor and restarted (no TMEM rewrite).
//
// Every mbarrier wait is made by one thread with a time limit and its outcome is shared through a block barrier, so
// a wait that runs out sets the error word and unwinds the whole CTA (copies drained, TMEM freed).
//
// Reference: the vendored decode / prefill kernels behind `csrc/glm_sparse_mla.cu:34-126` (bf16 `mma.sync` on expanded
// rows, split-K over the selected rows + combine).
#include "sparse_mla.cuh"
#include "tcgen05.cuh"

#include <cuda_fp8.h>

namespace {

constexpr int R = 512, NG = 4, GS = 128, DR = 64, ROW_BYTES = R + 4 * NG + 2 * DR;   // 656
constexpr int TILE = 128, NH = 8, NCOL = 2 * NH, THREADS = 256, HPT = NH / 2, ROWS_PER_WARP = TILE / (THREADS / 32);
constexpr int K8_TILE = TILE * GS;               // 16384: one code group of one key tile
constexpr int STAGE_K8 = NG * K8_TILE;           // 65536
constexpr int KR_TILE = TILE * 2 * DR;           // 16384
constexpr int B_TILE = NCOL * 128;               // 2048: a 16-row B operand with 128-byte rows
constexpr float RAISE = 8.f;                     // log2 units: exponentials stay below 2^8
constexpr float HEADROOM = 6.f;                  // a raised reference sits this far below the largest value seen: the two-term
                                                 // e4m3 form of P resolves 2^-13, i.e. 2^-19 of the row maximum
constexpr uint32_t TMEM_COLS = 256, COL_S = 0, COL_O = 96;

constexpr int MAX_TOPK = 2048;
constexpr int MAX_HEADS = 128;               // any head count in groups of 8 (each group gathers the rows again)

struct Smem {
    static constexpr int K8 = 0;
    static constexpr int KR = K8 + STAGE_K8;                // 65536
    static constexpr int SC = KR + KR_TILE;                 // 81920
    static constexpr int Q8 = SC + TILE * 16;               // 83968
    static constexpr int QR = Q8 + NG * B_TILE;             // 92160
    static constexpr int P = QR + B_TILE;                   // 94208
    static constexpr int SLOTS = P + NG * B_TILE;           // 102400: the token's slots (-1 = no row)
    static constexpr int INVQ = SLOTS + MAX_TOPK * 4;       // 110592
    static constexpr int MREF = INVQ + NH * 4;
    static constexpr int WRED = MREF + NH * 4;              // [4][NH]
    static constexpr int BARS = WRED + 4 * NH * 4;
    static constexpr int TOTAL = BARS + 2 * 8 + 16;
};
constexpr int SMEM_BYTES = Smem::TOTAL + 1024;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(tc::smem_u32(smem_dst)), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// two floats -> two e4m3 codes (a in the low byte), saturating
__device__ __forceinline__ uint32_t to_e4m3x2(float a, float b) {
    return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
}
// hardware approximations (2 ulp class): inputs here are finite and in range
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float2 from_e4m3x2(uint32_t v) { return e4m3x2_to_float2((uint16_t)v); }

// One thread waits (bounded); everybody learns the outcome.
__device__ __forceinline__ bool cta_wait(uint64_t* bar, uint32_t parity) {
    bool r = true;
    if (threadIdx.x == 0) r = tc::mbar_wait(bar, parity);
    r = __syncthreads_and(r);
    tc::fence_after_sync();
    return r;
}

__global__ void __launch_bounds__(THREADS, 2) sparse_mla_tc_kernel(SparseMlaParams p, int T, int head_groups) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sK8 = smem + Smem::K8;
    uint8_t* sKR = smem + Smem::KR;
    uint8_t* sSC = smem + Smem::SC;
    uint8_t* sQ8 = smem + Smem::Q8;
    uint8_t* sQR = smem + Smem::QR;
    uint8_t* sP = smem + Smem::P;
    int* s_slots = reinterpret_cast<int*>(smem + Smem::SLOTS);
    float* s_invq = reinterpret_cast<float*>(smem + Smem::INVQ);
    float* s_mref = reinterpret_cast<float*>(smem + Smem::MREF);
    float* s_wred = reinterpret_cast<float*>(smem + Smem::WRED);
    uint64_t* bar_s = reinterpret_cast<uint64_t*>(smem + Smem::BARS);
    uint64_t* bar_pv = bar_s + 1;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bar_pv + 1);

    // thread = (key of the tile | latent dim of a group, half of the heads): both halves of the block read the same
    // TMEM lanes (lane quarter = warp % 4) and different columns
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int key = tid & (TILE - 1), wq = warp & 3, hb = (tid >> 7) * HPT;
    if (tid == 0) {
        tc::mbar_init(bar_s, 1);
        tc::mbar_init(bar_pv, 1);
        tc::mbar_fence_init();
    }
    if (warp == 0) {
        tc::tmem_alloc(tmem_holder, TMEM_COLS);
        tc::tmem_relinquish();
    }
    // rows 8 .. 15 of the rope query operand stay zero for the whole kernel
    for (int i = tid; i < B_TILE / 16; i += THREADS) reinterpret_cast<uint4*>(sQR)[i] = make_uint4(0u, 0u, 0u, 0u);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    const uint32_t t_lane = tmem_base + ((uint32_t)(wq * 32) << 16);
    pdl_grid_sync();

    constexpr uint32_t IDESC_S = tc::idesc_f8(TILE, NCOL);
    constexpr uint32_t IDESC_R = tc::idesc_f16(TILE, NCOL, 1);
    constexpr uint32_t IDESC_PV = tc::idesc_f8(GS, NCOL) | tc::IDESC_A_MN_MAJOR;
    const float qk = p.sm_scale * 1.4426950408889634f;            // scores in log2 units
    uint32_t n_s = 0, n_pv = 0;                                    // phases of the two barriers consumed so far
    bool ok = true;

    // a warp copies 16 whole rows of the tile; per-lane parts of the addresses are fixed
    uint8_t* const g_dst = sK8 + (lane >> 3) * K8_TILE + warp * ROWS_PER_WARP * 128;
    uint8_t* const g_tail = lane == 0 ? sSC + warp * ROWS_PER_WARP * 16 : sKR + warp * ROWS_PER_WARP * 128;
    const int g_tail_pitch = lane == 0 ? 16 : 128;
    const uint8_t* const g_src = p.kv_cache + lane * 16;
    auto gather = [&](int tile) {
        const int* sl = s_slots + tile * TILE + warp * ROWS_PER_WARP;
#pragma unroll
        for (int r = 0; r < ROWS_PER_WARP; ++r) {
            const int slot = sl[r];
            const uint32_t sz = slot >= 0 ? 16u : 0u;
            const uint8_t* src = g_src + (size_t)(slot >= 0 ? slot : 0) * ROW_BYTES;
            cp_async16(g_dst + r * 128 + (((lane & 7) ^ (r & 7)) << 4), src, sz);
            if (lane < 9)                                          // piece 0 of the tail: scales; pieces 1 .. 8: rope
                cp_async16(g_tail + r * g_tail_pitch + (lane == 0 ? 0 : (((lane - 1) ^ (r & 7)) << 4)), src + R, sz);
        }
        cp_async_commit();
    };

    // work item = (query token, head group, key split); with one split the item writes the final bf16 output, with
    // several (decode) its normalised fp32 partial and log-sum-exp, which the merge kernel combines
    const int items = T * head_groups * p.splits;
    for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const int split = item % p.splits, th = item / p.splits;
        const int t = th / head_groups, h0 = (th % head_groups) * NH, nh = min(NH, p.h - h0);
        const int Lt = min(p.lengths[t], p.topk);
        const int per = (Lt + p.splits - 1) / p.splits;
        const int j_begin = min(Lt, split * per);
        const int L = min(Lt, j_begin + per) - j_begin;            // keys of this item
        const int* slots = p.slots + (size_t)t * p.topk + j_begin;
        const int ntiles = (L + TILE - 1) / TILE;
        __syncthreads();                                           // the previous item is done with Q, the reference and the sums

        // this warp's query head: its loads are in flight while the slots arrive
        uint4 qa = make_uint4(0u, 0u, 0u, 0u), qb = qa, qr4 = qa;
        if (warp < nh) {
            const uint4* src = reinterpret_cast<const uint4*>(p.q_abs + ((size_t)t * p.h + h0 + warp) * R + lane * 16);
            qa = __ldg(src); qb = __ldg(src + 1);
            if (lane < 8) qr4 = __ldg(reinterpret_cast<const uint4*>(p.q_pe + ((size_t)t * p.h + h0 + warp) * DR + lane * 8));
        }
        // the token's slots, padded with -1 to whole tiles
        for (int j = tid; j < ntiles * TILE; j += THREADS) {
            int sl = j < L ? slots[j] : -1;
            if (sl >= 0 && p.num_slots != 0 && !guard_ok(p.guard, 14, sl, p.num_slots)) sl = -1;
            s_slots[j] = sl;
        }
        __syncthreads();
        if (ntiles > 0) gather(0);                                 // in flight while the query operands are prepared
        // ---- query operands: one head per warp; lane = 16 latent values = one 16-byte piece of e4m3 codes ----
        {
            const int hh = warp;
            uint4 hi = make_uint4(0u, 0u, 0u, 0u), lo = hi;
            float inv = 1.f;
            if (hh < nh) {
                const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                float v[16];
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float2 f = bf162_to_f2(w[i]);
                    v[2 * i] = f.x * qk; v[2 * i + 1] = f.y * qk;
                    amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
                }
                amax = warp_max(amax);
                // largest power of two that keeps amax * qs <= 448
                float qs = 1.f;
                if (amax > 0.f) {
                    const float x = fminf(fmaxf(448.f / amax, 1e-30f), 1e30f);
                    qs = __uint_as_float(__float_as_uint(x) & 0x7f800000u);
                }
                inv = 1.f / qs;
                uint32_t hw4[4], lw4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t hword = 0u, lword = 0u;
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const float x0 = v[4 * i + 2 * k] * qs, x1 = v[4 * i + 2 * k + 1] * qs;
                        const uint32_t hp = to_e4m3x2(x0, x1);
                        const float2 back = from_e4m3x2(hp);
                        const uint32_t lp = to_e4m3x2((x0 - back.x) * 16.f, (x1 - back.y) * 16.f);
                        hword |= hp << (16 * k);
                        lword |= lp << (16 * k);
                    }
                    hw4[i] = hword; lw4[i] = lword;
                }
                hi = make_uint4(hw4[0], hw4[1], hw4[2], hw4[3]);
                lo = make_uint4(lw4[0], lw4[1], lw4[2], lw4[3]);
            }
            uint8_t* q8 = sQ8 + (lane >> 3) * B_TILE;
            const int cc = lane & 7;
            *reinterpret_cast<uint4*>(q8 + hh * 128 + ((cc ^ (hh & 7)) << 4)) = hi;
            *reinterpret_cast<uint4*>(q8 + (NH + hh) * 128 + ((cc ^ ((NH + hh) & 7)) << 4)) = lo;
            if (lane < 8) {
                uint4 rv = make_uint4(0u, 0u, 0u, 0u);
                if (hh < nh) {
                    const uint32_t w[4] = {qr4.x, qr4.y, qr4.z, qr4.w};
                    uint32_t o[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = bf162_to_f2(w[i]);
                        o[i] = f2_to_bf162(f.x * qk, f.y * qk);
                    }
                    rv = make_uint4(o[0], o[1], o[2], o[3]);
                }
                *reinterpret_cast<uint4*>(sQR + hh * 128 + ((lane ^ (hh & 7)) << 4)) = rv;
            }
            if (lane == 0) { s_invq[hh] = inv; s_mref[hh] = -INFINITY; }
        }

        float o_reg[NG][2][HPT];                                   // [group][hi | lo term][head of this thread]
#pragma unroll
        for (int g = 0; g < NG; ++g)
#pragma unroll
            for (int hh = 0; hh < HPT; ++hh) o_reg[g][0][hh] = o_reg[g][1][hh] = 0.f;
        float lsum[HPT];
#pragma unroll
        for (int hh = 0; hh < HPT; ++hh) lsum[hh] = 0.f;
        bool have_acc = false;
        auto fold_acc = [&]() {                                    // accumulators (dim `key` of each group) into registers
            uint32_t acc[NG][2][HPT];
#pragma unroll
            for (int g = 0; g < NG; ++g) {
                tc::tmem_ld_32x4(t_lane + COL_O + g * NCOL + hb, acc[g][0]);
                tc::tmem_ld_32x4(t_lane + COL_O + g * NCOL + NH + hb, acc[g][1]);
            }
            tc::tmem_ld_wait();
#pragma unroll
            for (int g = 0; g < NG; ++g)
#pragma unroll
                for (int hh = 0; hh < HPT; ++hh) {
                    o_reg[g][0][hh] += __uint_as_float(acc[g][0][hh]);
                    o_reg[g][1][hh] += __uint_as_float(acc[g][1][hh]);
                }
        };

        __syncthreads();                                           // query operands, reference
        for (int i = 0; i < ntiles && ok; ++i) {
            if (i > 0) gather(i);                                  // the previous tile's value product has been waited for
            cp_async_wait_all();
            tc::fence_proxy_async_smem();                          // this tile's rows (and, first time, the query operands)
            __syncthreads();
            if (tid == 0) {
                tc::fence_after_sync();
                const uint32_t a8 = tc::smem_u32(sK8), ar = tc::smem_u32(sKR);
                const uint32_t q8 = tc::smem_u32(sQ8), qr = tc::smem_u32(sQR);
#pragma unroll
                for (int g = 0; g < NG; ++g)
#pragma unroll
                    for (int ks = 0; ks < GS / 32; ++ks)
                        tc::mma_f8_ss(tmem_base + COL_S + g * NCOL, tc::smem_desc_sw128(a8 + g * K8_TILE + ks * 32),
                                      tc::smem_desc_sw128(q8 + g * B_TILE + ks * 32), IDESC_S, ks > 0 ? 1u : 0u);
#pragma unroll
                for (int ks = 0; ks < DR / 16; ++ks)
                    tc::mma_f16_ss(tmem_base + COL_S + NG * NCOL, tc::smem_desc_sw128(ar + ks * 32), tc::smem_desc_sw128(qr + ks * 32),
                                   IDESC_R, ks > 0 ? 1u : 0u);
                tc::mma_commit(bar_s);
            }
            ok = cta_wait(bar_s, n_s & 1);
            ++n_s;
            if (!ok) { if (tid == 0) atomicExch(p.err, 32); break; }

            // ---- scores of key `key` of the tile for this thread's four heads ----
            float u[HPT];
            float4 sc;
            float inv_scmax;
            {
                uint32_t dh[NG][HPT], dl[NG][HPT], dr[HPT];
#pragma unroll
                for (int g = 0; g < NG; ++g) {
                    tc::tmem_ld_32x4(t_lane + COL_S + g * NCOL + hb, dh[g]);
                    tc::tmem_ld_32x4(t_lane + COL_S + g * NCOL + NH + hb, dl[g]);
                }
                tc::tmem_ld_32x4(t_lane + COL_S + NG * NCOL + hb, dr);
                tc::tmem_ld_wait();
                sc = *reinterpret_cast<const float4*>(sSC + key * 16);
                const float scmax = fmaxf(fmaxf(fmaxf(sc.x, sc.y), fmaxf(sc.z, sc.w)), 1e-30f);
                const float lsc = lg2_approx(scmax);
                inv_scmax = __frcp_rn(scmax);
                const bool valid = s_slots[i * TILE + key] >= 0;
                const float scs[NG] = {sc.x, sc.y, sc.z, sc.w};
                const float4 iq = *reinterpret_cast<const float4*>(s_invq + hb);
                const float iqs[HPT] = {iq.x, iq.y, iq.z, iq.w};
#pragma unroll
                for (int hh = 0; hh < HPT; ++hh) {
                    float lat = 0.f;
#pragma unroll
                    for (int g = 0; g < NG; ++g)
                        lat = fmaf(scs[g], fmaf(__uint_as_float(dl[g][hh]), 0.0625f, __uint_as_float(dh[g][hh])), lat);
                    const float sv = fmaf(lat, iqs[hh], __uint_as_float(dr[hh]));
                    u[hh] = valid ? sv + lsc : -INFINITY;
                }
            }
            // ---- raise the reference when a value exceeds it by more than 2^RAISE ----
            float mref[HPT];
            {
                const float4 m4 = *reinterpret_cast<const float4*>(s_mref + hb);
                mref[0] = m4.x; mref[1] = m4.y; mref[2] = m4.z; mref[3] = m4.w;
            }
            bool raise = false;
#pragma unroll
            for (int hh = 0; hh < HPT; ++hh) raise |= u[hh] > mref[hh] + RAISE;
            if (__syncthreads_or(raise)) {
#pragma unroll
                for (int hh = 0; hh < HPT; ++hh) {
                    const float m = warp_max(u[hh]);
                    if (lane == 0) s_wred[wq * NH + hb + hh] = m;
                }
                __syncthreads();
                float f[HPT];
#pragma unroll
                for (int hh = 0; hh < HPT; ++hh) {
                    const int h = hb + hh;
                    const float tmax = fmaxf(fmaxf(s_wred[h], s_wred[NH + h]), fmaxf(s_wred[2 * NH + h], s_wred[3 * NH + h]));
                    const float mn = fmaxf(mref[hh], tmax - HEADROOM);
                    f[hh] = mn == -INFINITY ? 1.f : exp2f(mref[hh] - mn);
                    mref[hh] = mn;
                }
                if (have_acc) {
                    fold_acc();
                    have_acc = false;
                }
#pragma unroll
                for (int g = 0; g < NG; ++g)
#pragma unroll
                    for (int hh = 0; hh < HPT; ++hh) { o_reg[g][0][hh] *= f[hh]; o_reg[g][1][hh] *= f[hh]; }
#pragma unroll
                for (int hh = 0; hh < HPT; ++hh) lsum[hh] *= f[hh];
                if (key == 0) *reinterpret_cast<float4*>(s_mref + hb) = make_float4(mref[0], mref[1], mref[2], mref[3]);
                // (the old reference lives in registers; the next read of s_mref is after the barrier that follows P)
            }
            // ---- P_g = exp2(u - ref) * scale[g] / scmax in two e4m3 terms: byte `key` of rows h and 8 + h of the B operand ----
            {
                const float r0 = sc.x * inv_scmax, r1 = sc.y * inv_scmax, r2 = sc.z * inv_scmax, r3 = sc.w * inv_scmax;
                uint8_t* pb = sP + (key & 15);
                const int chunk = key >> 4;
#pragma unroll
                for (int hh = 0; hh < HPT; ++hh) {
                    const int h = hb + hh;
                    const float e = u[hh] == -INFINITY ? 0.f : ex2_approx(u[hh] - mref[hh]);      // masked key: 0
                    lsum[hh] = fmaf(e, inv_scmax, lsum[hh]);
                    const float p0 = e * r0, p1 = e * r1, p2 = e * r2, p3 = e * r3;
                    const uint32_t h01 = to_e4m3x2(p0, p1), h23 = to_e4m3x2(p2, p3);
                    const float2 b01 = from_e4m3x2(h01), b23 = from_e4m3x2(h23);
                    const uint32_t l01 = to_e4m3x2((p0 - b01.x) * 16.f, (p1 - b01.y) * 16.f);
                    const uint32_t l23 = to_e4m3x2((p2 - b23.x) * 16.f, (p3 - b23.y) * 16.f);
                    // rows h and 8 + h have the same swizzle phase (h & 7)
                    uint8_t* ph = pb + h * 128 + ((chunk ^ (h & 7)) << 4);
                    ph[0 * B_TILE] = (uint8_t)(h01 & 0xffu);
                    ph[1 * B_TILE] = (uint8_t)(h01 >> 8);
                    ph[2 * B_TILE] = (uint8_t)(h23 & 0xffu);
                    ph[3 * B_TILE] = (uint8_t)(h23 >> 8);
                    ph[0 * B_TILE + NH * 128] = (uint8_t)(l01 & 0xffu);
                    ph[1 * B_TILE + NH * 128] = (uint8_t)(l01 >> 8);
                    ph[2 * B_TILE + NH * 128] = (uint8_t)(l23 & 0xffu);
                    ph[3 * B_TILE + NH * 128] = (uint8_t)(l23 >> 8);
                }
            }
            tc::fence_proxy_async_smem();
            tc::fence_before_sync();                               // the score accumulators have been read
            __syncthreads();
            if (tid == 0) {
                tc::fence_after_sync();
                const uint32_t a8 = tc::smem_u32(sK8), pb = tc::smem_u32(sP);
#pragma unroll
                for (int g = 0; g < NG; ++g)
#pragma unroll
                    for (int ks = 0; ks < TILE / 32; ++ks)
                        tc::mma_f8_ss(tmem_base + COL_O + g * NCOL, tc::smem_desc_sw128(a8 + g * K8_TILE + ks * 32 * 128),
                                      tc::smem_desc_sw128(pb + g * B_TILE + ks * 32), IDESC_PV, (have_acc || ks > 0) ? 1u : 0u);
                tc::mma_commit(bar_pv);
            }
            have_acc = true;
            ok = cta_wait(bar_pv, n_pv & 1);                       // the key tile and P are free again
            ++n_pv;
            if (!ok) { if (tid == 0) atomicExch(p.err, 33); break; }
        }
        if (!ok) break;
        if (have_acc) {
            fold_acc();
            tc::fence_before_sync();
        }
        // ---- softmax denominators, output ----
#pragma unroll
        for (int hh = 0; hh < HPT; ++hh) {
            const float x = warp_sum(lsum[hh]);
            if (lane == 0) s_wred[wq * NH + hb + hh] = x;
        }
        __syncthreads();
#pragma unroll
        for (int hh = 0; hh < HPT; ++hh) {
            const int h = hb + hh;
            if (h < nh) {
                const float l = s_wred[h] + s_wred[NH + h] + s_wred[2 * NH + h] + s_wred[3 * NH + h];
                const float inv = l > 0.f ? 1.f / l : 0.f;
                if (p.o_final != nullptr) {
                    bf16* o = p.o_final + ((size_t)t * p.h + h0 + h) * R + key;
#pragma unroll
                    for (int g = 0; g < NG; ++g) o[g * GS] = __float2bfloat16(fmaf(o_reg[g][1][hh], 0.0625f, o_reg[g][0][hh]) * inv);
                } else {
                    float* o = p.o_part + (((size_t)t * p.h + h0 + h) * p.splits + split) * R + key;
#pragma unroll
                    for (int g = 0; g < NG; ++g) o[g * GS] = fmaf(o_reg[g][1][hh], 0.0625f, o_reg[g][0][hh]) * inv;
                }
            }
        }
        if (tid < nh) {
            const float l = s_wred[tid] + s_wred[NH + tid] + s_wred[2 * NH + tid] + s_wred[3 * NH + tid];
            const float lse = l > 0.f ? (s_mref[tid] + log2f(l)) * 0.6931471805599453f : -INFINITY;
            if (p.o_final == nullptr) p.lse_part[((size_t)t * p.h + h0 + tid) * p.splits + split] = lse;
            else if (p.lse_final != nullptr) p.lse_final[(size_t)t * p.h + h0 + tid] = lse;
        }
    }
    cp_async_wait_all();
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

int g_mla_tcgen05 = 3;            // bit 0: launches that write the final output (prefill); bit 1: key-split launches (decode)

}  // namespace

int sparse_mla_tcgen05(const SparseMlaParams* p, int T, cudaStream_t s) {
    const bool direct = p->o_final != nullptr;
    if (p->err == nullptr || !(g_mla_tcgen05 & (direct ? 1 : 2))) return -2;
    if (direct ? p->splits != 1 : (p->splits < 1 || p->o_part == nullptr || p->lse_part == nullptr)) return -2;
    if (p->R != R || p->group != GS || p->Dr != DR || p->h > MAX_HEADS || p->topk <= 0 || p->topk > MAX_TOPK) return -2;
    if (((uintptr_t)p->q_abs & 15) != 0 || ((uintptr_t)p->q_pe & 15) != 0 || ((uintptr_t)p->kv_cache & 15) != 0) return -2;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(sparse_mla_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        attr_done = true;
    }
    const int head_groups = (p->h + NH - 1) / NH;
    const long long items = (long long)T * head_groups * p->splits;
    const int max_ctas = 2 * 148;
    sl_launch(sparse_mla_tc_kernel, dim3((unsigned)(items < max_ctas ? items : max_ctas)), THREADS, SMEM_BYTES, s, *p, T, head_groups);
    return SL_LAUNCH_CHECK();
}

// Which launches take the tcgen05 kernel: 0 none (the mma.sync kernels everywhere, comparison runs), 1 those that write the
// final output (prefill), 3 (default) also the key-split launches of decode.
SL_API void sl_sparse_mla_set_tcgen05(int mode) { g_mla_tcgen05 = mode; }

// 1 when a key-split launch with these row parameters takes the tcgen05 kernel (one 128-key tile per split is its unit of work).
SL_API int sl_sparse_mla_tcgen05_decode_ok(int R_, int group, int Dr, int h, int topk) {
    return ((g_mla_tcgen05 & 2) && R_ == R && group == GS && Dr == DR && h <= MAX_HEADS && topk > 0 && topk <= MAX_TOPK) ? 1 : 0;
}
