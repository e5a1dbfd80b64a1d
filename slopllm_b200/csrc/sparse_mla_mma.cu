// Sparse MLA flash attention on the tensor cores (decode and prefill): per (key split, group of
// 16 heads, query token) one CTA gathers its selected packed rows (fp8 latent x per-group scale,
// bf16 rope), expands them to f16 in shared memory, computes S = Q K^T and O += P V with
// `mma.sync.m16n8k16` (fp32 accumulation, online softmax) and emits a partial (o, lse) that the
// combine kernel (or the cross-rank merge under context parallelism) finishes.
//
// Covers what the reference gets from the vendored `sparse_mla_sm120` decode / prefill kernels
// (`csrc/glm_sparse_mla.cu:34-126`): split-K over the top-k rows, mid_out / mid_lse + combine.
#include "sparse_mla.cuh"

#include <type_traits>

namespace {

using Params = SparseMlaParams;

constexpr int HB = 16;        // heads per CTA (one MMA row tile)
constexpr int KC = 64;        // keys per chunk (8 warps x 8 keys)

__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(a));
}

// grid (splits, ceil(h / 16), T); block 256.
// Shared: Q [16][DP] f16, K [64][DP] f16 (DP = R + Dr + 8 halves: rows 16-byte aligned, bank-skewed),
// P [16][72] f16, row statistics.
__global__ void __launch_bounds__(256) sparse_mla_mma_kernel(Params p) {
    pdl_grid_sync();
    extern __shared__ __align__(16) unsigned char smraw[];
    const int D = p.R + p.Dr, DP = D + 8;
    __half* qs = reinterpret_cast<__half*>(smraw);            // HB * DP
    __half* ks = qs + HB * DP;                                // KC * DP
    __half* ps = ks + KC * DP;                                // HB * 72
    float* wmax = reinterpret_cast<float*>(ps + HB * 72);     // [8 warps][16 rows]
    float* wsum = wmax + 8 * HB;                              // [8 warps][16 rows]
    float* row_m = wsum + 8 * HB;                             // [16] running max
    float* row_l = row_m + HB;                                // [16] running sum
    float* row_a = row_l + HB;                                // [16] rescale of this chunk
    int* s_slots = reinterpret_cast<int*>(row_a + HB);        // [2][64] slots of the current / next chunk

    const int split = blockIdx.x, hg = blockIdx.y, t = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, c = lane & 3;
    const int L = p.lengths[t];
    const int per = (L + p.splits - 1) / p.splits;
    const int j_begin = min(L, split * per), j_end = min(L, j_begin + per);
    const int h0 = hg * HB, nh = min(HB, p.h - h0);
    const int ngroups = p.R / p.group;
    const int row_bytes = p.R + 4 * ngroups + 2 * p.Dr;
    const int words = row_bytes / 4;
    // 16-byte gather path: every field boundary of the row falls on a 16-byte boundary
    const bool vec16 = row_bytes % 16 == 0 && p.R % 16 == 0 && (4 * ngroups) % 16 == 0 && p.group % 16 == 0 &&
                       KC * (row_bytes / 16) <= 12 * 256;
    const int* slots = p.slots + (size_t)t * p.topk;

    // Q (pre-multiplied by the softmax scale) as f16; rows >= nh are zero
    for (int i = tid; i < HB * (D / 2); i += blockDim.x) {
        const int hh = i / (D / 2), d = (i % (D / 2)) * 2;
        float2 v = make_float2(0.f, 0.f);
        if (hh < nh) {
            const uint32_t u = d < p.R ? *reinterpret_cast<const uint32_t*>(p.q_abs + ((size_t)t * p.h + h0 + hh) * p.R + d)
                                       : *reinterpret_cast<const uint32_t*>(p.q_pe + ((size_t)t * p.h + h0 + hh) * p.Dr + (d - p.R));
            v = bf162_to_f2(u);
        }
        *reinterpret_cast<__half2*>(qs + hh * DP + d) = __floats2half2_rn(v.x * p.sm_scale, v.y * p.sm_scale);
    }
    if (tid < HB) { row_m[tid] = -INFINITY; row_l[tid] = 0.f; }

    // output accumulators: warp w owns dims [w*R/8, (w+1)*R/8), up to 8 n-tiles of 8 dims
    const int dims_per_warp = p.R / 8, ntiles = dims_per_warp / 8;
    float oacc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;

    // a slot outside the cache is recorded and replaced by row 0 (its score is garbage, the step is reported as failed)
    auto checked_slot = [&](int s) { return (p.num_slots == 0 || guard_ok(p.guard, 11, s, p.num_slots)) ? s : 0; };
    // 16-byte gather path: the rows of chunk c+1 are loaded into registers while chunk c is multiplied, so the
    // gather latency overlaps the tensor-core phases (a thread's loads are all issued before their first use).
    constexpr int MAXLD = 12;
    uint4 buf[MAXLD];
    float scl[MAXLD];
    const int chunks = row_bytes / 16;
    auto issue_loads = [&](int c0n, const int* sl) {
        const int kcn = min(KC, j_end - c0n), total = kcn * chunks;
#pragma unroll
        for (int n = 0; n < MAXLD; ++n) {
            const int i = tid + n * 256;
            if (i < total) {
                const int j = i / chunks, byte = (i % chunks) * 16;
                const uint8_t* row = p.kv_cache + (size_t)sl[j] * row_bytes;
                buf[n] = ldg_nc_16(row + byte);
                scl[n] = byte < p.R ? *reinterpret_cast<const float*>(row + p.R + 4 * (byte / p.group)) : 0.f;
            }
        }
    };
    int* s_slots2 = s_slots + KC;                               // second slot buffer (pipelined path)
    if (vec16 && j_begin < j_end) {
        if (tid < KC) s_slots[tid] = tid < min(KC, j_end - j_begin) ? checked_slot(slots[j_begin + tid]) : 0;
        __syncthreads();
        issue_loads(j_begin, s_slots);
    }
    int parity = 0;

    for (int c0 = j_begin; c0 < j_end; c0 += KC) {
        const int kc = min(KC, j_end - c0);
        __syncthreads();
        // ---- gather + expand kc rows ----
        if (vec16) {
            const int total = kc * chunks;
#pragma unroll
            for (int n = 0; n < MAXLD; ++n) {
                const int i = tid + n * 256;
                if (i < total) {
                    const int j = i / chunks, byte = (i % chunks) * 16;
                    const uint32_t w4[4] = {buf[n].x, buf[n].y, buf[n].z, buf[n].w};
                    if (byte < p.R) {
                        uint32_t o[8];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float2 a = e4m3x2_to_float2((uint16_t)(w4[q] & 0xffffu)), b = e4m3x2_to_float2((uint16_t)(w4[q] >> 16));
                            __half2 lo = __floats2half2_rn(a.x * scl[n], a.y * scl[n]), hi = __floats2half2_rn(b.x * scl[n], b.y * scl[n]);
                            o[2 * q] = *reinterpret_cast<uint32_t*>(&lo);
                            o[2 * q + 1] = *reinterpret_cast<uint32_t*>(&hi);
                        }
                        uint4* dst = reinterpret_cast<uint4*>(ks + j * DP + byte);
                        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
                        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
                    } else if (byte >= p.R + 4 * ngroups) {
                        const int d = p.R + (byte - p.R - 4 * ngroups) / 2;
                        uint32_t o[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float2 f = bf162_to_f2(w4[q]);
                            __half2 hv = __floats2half2_rn(f.x, f.y);
                            o[q] = *reinterpret_cast<uint32_t*>(&hv);
                        }
                        *reinterpret_cast<uint4*>(ks + j * DP + d) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                }
            }
            // slots of the next chunk, then its loads (in flight during this chunk's MMAs)
            const int c0n = c0 + KC;
            int* sl_next = parity ? s_slots : s_slots2;
            if (c0n < j_end && tid < KC) sl_next[tid] = tid < min(KC, j_end - c0n) ? checked_slot(slots[c0n + tid]) : 0;
            __syncthreads();
            if (c0n < j_end) issue_loads(c0n, sl_next);
            parity ^= 1;
        } else {
        if (tid < KC) s_slots[tid] = tid < kc ? checked_slot(slots[c0 + tid]) : 0;
        __syncthreads();
        for (int i = tid; i < KC * words; i += blockDim.x) {
            const int j = i / words, wd = i % words, byte = wd * 4;
            if (j < kc) {
                const uint8_t* row = p.kv_cache + (size_t)s_slots[j] * row_bytes;
                const uint32_t u = *reinterpret_cast<const uint32_t*>(row + byte);
                if (byte < p.R) {
                    const float sc = *reinterpret_cast<const float*>(row + p.R + 4 * (byte / p.group));
                    const float2 a = e4m3x2_to_float2((uint16_t)(u & 0xffffu)), b = e4m3x2_to_float2((uint16_t)(u >> 16));
                    __half2 lo = __floats2half2_rn(a.x * sc, a.y * sc), hi = __floats2half2_rn(b.x * sc, b.y * sc);
                    uint2 o;
                    o.x = *reinterpret_cast<uint32_t*>(&lo);
                    o.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(ks + j * DP + byte) = o;
                } else if (byte >= p.R + 4 * ngroups) {
                    const int d = p.R + (byte - p.R - 4 * ngroups) / 2;
                    const float2 f = bf162_to_f2(u);
                    *reinterpret_cast<__half2*>(ks + j * DP + d) = __floats2half2_rn(f.x, f.y);
                }
            }
        }
        }
        // rows beyond kc contribute p = 0; keep them finite so that 0 * v stays 0
        for (int i = tid; i < (KC - kc) * (D / 2); i += blockDim.x) {
            const int j = kc + i / (D / 2), d2 = i % (D / 2);
            reinterpret_cast<uint32_t*>(ks + j * DP)[d2] = 0u;
        }
        __syncthreads();
        // ---- S = Q K^T : warp w -> keys 8w .. 8w+7 ----
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        for (int k0 = 0; k0 < D; k0 += 16) {
            uint32_t a[4];
            // A tile rows 0..15, cols k0..k0+15: lanes 0-15 -> rows, lanes 16-31 -> rows with col + 8
            ldmatrix_x4(a, qs + (lane & 15) * DP + k0 + (lane >> 4) * 8);
            const __half* kr = ks + (warp * 8 + g) * DP + k0 + 2 * c;
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kr), b1 = *reinterpret_cast<const uint32_t*>(kr + 8);
            mma16816(s, a, b0, b1);
        }
        // s[0]:(head g, key 2c) s[1]:(g, 2c+1) s[2]:(g+8, 2c) s[3]:(g+8, 2c+1)
        const int key0 = warp * 8 + 2 * c;
        if (key0 >= kc) { s[0] = -INFINITY; s[2] = -INFINITY; }
        if (key0 + 1 >= kc) { s[1] = -INFINITY; s[3] = -INFINITY; }
        float m0 = fmaxf(s[0], s[1]), m1 = fmaxf(s[2], s[3]);
        m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 1)); m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 2));
        m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 1)); m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 2));
        if (c == 0) { wmax[warp * HB + g] = m0; wmax[warp * HB + g + 8] = m1; }
        __syncthreads();
        if (tid < HB) {
            float mx = row_m[tid];
            const float old = mx;
#pragma unroll
            for (int w = 0; w < 8; ++w) mx = fmaxf(mx, wmax[w * HB + tid]);
            row_a[tid] = (old == -INFINITY) ? 0.f : __expf(old - mx);
            row_m[tid] = mx;
        }
        __syncthreads();
        const float mn0 = row_m[g], mn1 = row_m[g + 8];
        float e[4];
        e[0] = (s[0] == -INFINITY) ? 0.f : __expf(s[0] - mn0);
        e[1] = (s[1] == -INFINITY) ? 0.f : __expf(s[1] - mn0);
        e[2] = (s[2] == -INFINITY) ? 0.f : __expf(s[2] - mn1);
        e[3] = (s[3] == -INFINITY) ? 0.f : __expf(s[3] - mn1);
        *reinterpret_cast<__half2*>(ps + g * 72 + key0) = __floats2half2_rn(e[0], e[1]);
        *reinterpret_cast<__half2*>(ps + (g + 8) * 72 + key0) = __floats2half2_rn(e[2], e[3]);
        float l0 = e[0] + e[1], l1 = e[2] + e[3];
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        if (c == 0) { wsum[warp * HB + g] = l0; wsum[warp * HB + g + 8] = l1; }
        __syncthreads();
        if (tid < HB) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) sum += wsum[w * HB + tid];
            row_l[tid] = row_l[tid] * row_a[tid] + sum;
        }
        // ---- O = O * alpha + P V : warp w -> dims [w*dims_per_warp, ...) ----
        const float a0 = row_a[g], a1 = row_a[g + 8];
#pragma unroll
        for (int i = 0; i < 8; ++i) { oacc[i][0] *= a0; oacc[i][1] *= a0; oacc[i][2] *= a1; oacc[i][3] *= a1; }
#pragma unroll
        for (int k0 = 0; k0 < KC; k0 += 16) {
            uint32_t a[4];
            ldmatrix_x4(a, ps + (lane & 15) * 72 + k0 + (lane >> 4) * 8);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (i < ntiles) {
                    uint32_t b0, b1;
                    // V[k = key k0 + (lane & 15)][n = dim0 .. dim0 + 7], transposed on load
                    ldmatrix_x2_trans(b0, b1, ks + (k0 + (lane & 15)) * DP + warp * dims_per_warp + i * 8);
                    mma16816(oacc[i], a, b0, b1);
                }
            }
        }
    }
    __syncthreads();
    // ---- write the normalised partial ----
    const float l0 = row_l[g], l1 = row_l[g + 8];
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (i < ntiles) {
            const int d = warp * dims_per_warp + i * 8 + 2 * c;
            if (g < nh) {
                float* o = p.o_part + (((size_t)t * p.h + h0 + g) * p.splits + split) * p.R + d;
                *reinterpret_cast<float2*>(o) = make_float2(oacc[i][0] * i0, oacc[i][1] * i0);
            }
            if (g + 8 < nh) {
                float* o = p.o_part + (((size_t)t * p.h + h0 + g + 8) * p.splits + split) * p.R + d;
                *reinterpret_cast<float2*>(o) = make_float2(oacc[i][2] * i1, oacc[i][3] * i1);
            }
        }
    }
    if (tid < nh) {
        const float l = row_l[tid];
        p.lse_part[((size_t)t * p.h + h0 + tid) * p.splits + split] = l > 0.f ? row_m[tid] + logf(l) : -INFINITY;
    }
}


// ---------------------------------------------------------------------------------------------------
// Transposed form (keys on the MMA M dimension, heads on N in tiles of 8) for the 656-byte cache row:
// 512 e4m3 latent values, 4 fp32 scales (one per 128 values), 64 bf16 rope values.
//
//   S^T[64 keys, 8 heads]   = K8[64, 576] Q^T[576, 8]    warp (mt, kh): 16 keys x 18 of the 36 k-steps
//   O^T[512 dims, 8 heads] += V8^T[512, 64] P'[64, 8]    warp w: 64 dims
//
// With 8 heads per rank (64 heads over 8 GPUs) no MMA row is padding, against half of them with heads on M.
// The latent part of a row stays in its e4m3 code values (exact in f16): the per-(key, group) scale is applied
// to the fp32 group sums of S and folded into P for the output product, so expanding a row is one convert per
// pair of elements.  The running maximum is a reference that is only raised when a score exceeds it by more
// than `kRaise` (one vote per chunk through the barrier that publishes P): exponentials stay below e^kRaise,
// and the common chunk has four barriers and no single-warp phase.  The row geometry is a compile-time
// constant: a warp gathers whole rows (lane = 16-byte piece of the latent part), so no index needs a division.
constexpr float kRaise = 6.f;
bool g_transposed_enabled = true;

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
// four e4m3 codes -> four halves (a: codes 0 and 1, b: codes 2 and 3)
__device__ __forceinline__ void e4m3x4_to_h2x2(uint32_t w, uint32_t& a, uint32_t& b) {
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %2; cvt.rn.f16x2.e4m3x2 %0, lo; cvt.rn.f16x2.e4m3x2 %1, hi; }"
        : "=r"(a), "=r"(b) : "r"(w));
}

namespace tk {                                   // geometry of the transposed kernel
constexpr int R = 512, GS = 128, NG = R / GS, DR = 64, D = R + DR, DP = D + 8;
constexpr int ROW_BYTES = R + 4 * NG + 2 * DR;   // 656
constexpr int TAIL = (4 * NG + 2 * DR) / 16;     // 16-byte pieces after the latent part: 1 of scales, 8 of rope
constexpr int ROWS_PER_WARP = KC / 8;            // 8
constexpr int TAIL_ITEMS = KC * TAIL;            // 576 = 2.25 per thread
constexpr int PS = KC + 8;                       // row stride of P in halves
constexpr int NSTEPS = D / 16, HALF = NSTEPS / 2, SPG = GS / 16, NOPE_STEPS = R / 16;
static_assert(R / 16 == 32, "one lane per 16-byte piece of the latent part");
static_assert(NSTEPS % 2 == 0 && R / 8 == 64, "");
}  // namespace tk

// grid (splits, ceil(h / (8 NT)), T); block 256.
template <int NT>
__global__ void __launch_bounds__(256) sparse_mla_mma_t_kernel(Params p) {
    using namespace tk;
    pdl_grid_sync();
    extern __shared__ __align__(16) unsigned char smraw[];
    constexpr int NH = 8 * NT;
    __half* qs = reinterpret_cast<__half*>(smraw);            // NH * DP
    __half* ks = qs + NH * DP;                                // KC * DP
    __half* ps = ks + KC * DP;                                // NH * PS
    float* sks = reinterpret_cast<float*>(ps + NH * PS);      // [KC][NG] group scales of the chunk's keys
    float4* xs = reinterpret_cast<float4*>(sks + KC * NG);    // [4][NT][32] S partial sums of the second k half
    float* wmax = reinterpret_cast<float*>(xs + 4 * NT * 32); // [4][NH]
    float* wl = wmax + 4 * NH;                                // [4][NH]
    float* row_m = wl + 4 * NH;                               // [NH] reference maximum
    int* s_slots = reinterpret_cast<int*>(row_m + NH);        // [2][KC]

    const int split = blockIdx.x, hg = blockIdx.y, t = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, c = lane & 3;
    const int mt = warp & 3, kh = warp >> 2;
    const int L = p.lengths[t];
    const int per = (L + p.splits - 1) / p.splits;
    const int j_begin = min(L, split * per), j_end = min(L, j_begin + per);
    const int h0 = hg * NH, nh = min(NH, p.h - h0);
    const int* slots = p.slots + (size_t)t * p.topk;

    for (int i = tid; i < NH * (D / 2); i += 256) {
        const int hh = i / (D / 2), d = (i % (D / 2)) * 2;
        float2 v = make_float2(0.f, 0.f);
        if (hh < nh) {
            const uint32_t u = d < R ? *reinterpret_cast<const uint32_t*>(p.q_abs + ((size_t)t * p.h + h0 + hh) * R + d)
                                     : *reinterpret_cast<const uint32_t*>(p.q_pe + ((size_t)t * p.h + h0 + hh) * DR + (d - R));
            v = bf162_to_f2(u);
        }
        *reinterpret_cast<__half2*>(qs + hh * DP + d) = __floats2half2_rn(v.x * p.sm_scale, v.y * p.sm_scale);
    }
    if (tid < NH) row_m[tid] = -INFINITY;

    const int grp_w = warp >> 1;                              // scale group of this warp's 64 output dims
    float oacc[4][NT][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) oacc[i][nt][0] = oacc[i][nt][1] = oacc[i][nt][2] = oacc[i][nt][3] = 0.f;
    float lsum[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) lsum[nt][0] = lsum[nt][1] = 0.f;

    auto checked_slot = [&](int s) { return (p.num_slots == 0 || guard_ok(p.guard, 12, s, p.num_slots)) ? s : 0; };
    // gather registers: the latent piece `lane` of this warp's 8 rows, and up to 3 of the chunk's 576 tail pieces
    uint4 nbuf[ROWS_PER_WARP], tbuf[3];
    auto issue_loads = [&](int kcn, const int* sl) {
#pragma unroll
        for (int r = 0; r < ROWS_PER_WARP; ++r) {
            const int row = warp * ROWS_PER_WARP + r;
            if (row < kcn) nbuf[r] = ldg_nc_16(p.kv_cache + (size_t)sl[row] * ROW_BYTES + lane * 16);
        }
#pragma unroll
        for (int n = 0; n < 3; ++n) {
            const int item = tid + n * 256, row = item / TAIL, q = item - row * TAIL;
            if (item < TAIL_ITEMS && row < kcn) tbuf[n] = ldg_nc_16(p.kv_cache + (size_t)sl[row] * ROW_BYTES + R + q * 16);
        }
    };
    int* s_slots2 = s_slots + KC;
    if (j_begin < j_end) {
        const int kc0 = min(KC, j_end - j_begin);
        if (tid < KC) s_slots[tid] = tid < kc0 ? checked_slot(slots[j_begin + tid]) : 0;
        __syncthreads();
        issue_loads(kc0, s_slots);
    }
    int parity = 0;
    const int keyA = 16 * mt + g, keyB = keyA + 8;
    const __half* arow = ks + (16 * mt + (lane & 15)) * DP + (lane >> 4) * 8;
    const __half* brow = qs + g * DP + 2 * c;
    const __half* vrow0 = ks + ((lane & 7) + ((lane >> 4) & 1) * 8) * DP + warp * 64 + ((lane >> 3) & 1) * 8;

    for (int c0 = j_begin; c0 < j_end; c0 += KC) {
        const int kc = min(KC, j_end - c0);
        __syncthreads();                                      // the previous chunk's products have read ks / ps / sks
        // ---- expand the prefetched rows: e4m3 codes -> f16, scales aside, rope bf16 -> f16; rows beyond kc are
        //      zero (their p is 0: values and scales must be finite so that 0 * v stays 0) ----
#pragma unroll
        for (int r = 0; r < ROWS_PER_WARP; ++r) {
            const int row = warp * ROWS_PER_WARP + r;
            uint4 lo = make_uint4(0u, 0u, 0u, 0u), hi = lo;
            if (row < kc) {
                const uint4 w = nbuf[r];
                e4m3x4_to_h2x2(w.x, lo.x, lo.y);
                e4m3x4_to_h2x2(w.y, lo.z, lo.w);
                e4m3x4_to_h2x2(w.z, hi.x, hi.y);
                e4m3x4_to_h2x2(w.w, hi.z, hi.w);
            }
            uint4* dst = reinterpret_cast<uint4*>(ks + row * DP + lane * 16);
            dst[0] = lo;
            dst[1] = hi;
        }
#pragma unroll
        for (int n = 0; n < 3; ++n) {
            const int item = tid + n * 256, row = item / TAIL, q = item - row * TAIL;
            if (item < TAIL_ITEMS) {
                const uint4 w = row < kc ? tbuf[n] : make_uint4(0u, 0u, 0u, 0u);
                if (q == 0) {
                    *reinterpret_cast<uint4*>(sks + row * NG) = w;
                } else {
                    const uint32_t w4[4] = {w.x, w.y, w.z, w.w};
                    uint32_t o[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = bf162_to_f2(w4[e]);
                        __half2 hv = __floats2half2_rn(f.x, f.y);
                        o[e] = *reinterpret_cast<uint32_t*>(&hv);
                    }
                    *reinterpret_cast<uint4*>(ks + row * DP + R + (q - 1) * 8) = make_uint4(o[0], o[1], o[2], o[3]);
                }
            }
        }
        const int c0n = c0 + KC, kcn = min(KC, j_end - c0n);
        int* sl_next = parity ? s_slots : s_slots2;
        if (c0n < j_end && tid < KC) sl_next[tid] = tid < kcn ? checked_slot(slots[c0n + tid]) : 0;
        __syncthreads();                                      // tile, scales and the next slot list are in place
        if (c0n < j_end) issue_loads(kcn, sl_next);           // in flight during this chunk's products
        parity ^= 1;

        // ---- S^T = K Q^T : warp (mt, kh) -> keys 16 mt .. 16 mt + 15, k-steps [18 kh, 18 kh + 18) ----
        float sacc[NT][4], acc[2][NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int q = 0; q < 4; ++q) sacc[nt][q] = acc[0][nt][q] = acc[1][nt][q] = 0.f;
        auto fold = [&](int grp) {                            // grp < 0: the rope part carries no scale
            const float fa = grp >= 0 ? sks[keyA * NG + grp] : 1.f, fb = grp >= 0 ? sks[keyB * NG + grp] : 1.f;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                sacc[nt][0] += (acc[0][nt][0] + acc[1][nt][0]) * fa;
                sacc[nt][1] += (acc[0][nt][1] + acc[1][nt][1]) * fa;
                sacc[nt][2] += (acc[0][nt][2] + acc[1][nt][2]) * fb;
                sacc[nt][3] += (acc[0][nt][3] + acc[1][nt][3]) * fb;
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[0][nt][q] = acc[1][nt][q] = 0.f;
            }
        };
        auto s_half = [&](auto KH) {
            constexpr int kh_ = decltype(KH)::value;
#pragma unroll
            for (int i = 0; i < HALF; ++i) {
                const int st = kh_ * HALF + i;
                if (i > 0 && st <= NOPE_STEPS && st % SPG == 0) fold(st / SPG - 1);
                uint32_t a[4];
                ldmatrix_x4(a, arow + st * 16);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const __half* br = brow + nt * 8 * DP + st * 16;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(br), b1 = *reinterpret_cast<const uint32_t*>(br + 8);
                    mma16816(acc[i & 1][nt], a, b0, b1);
                }
            }
            constexpr int last = kh_ * HALF + HALF - 1;
            fold(last < NOPE_STEPS ? last / SPG : -1);
        };
        if (kh == 0) s_half(std::integral_constant<int, 0>{}); else s_half(std::integral_constant<int, 1>{});
        if (kh == 1) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) xs[(mt * NT + nt) * 32 + lane] = make_float4(sacc[nt][0], sacc[nt][1], sacc[nt][2], sacc[nt][3]);
        }
        __syncthreads();
        // ---- P = exp(S - reference) on the warps of the first k half ----
        float e[NT][4];
        int raise = 0;
        if (kh == 0) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float4 o = xs[(mt * NT + nt) * 32 + lane];
                sacc[nt][0] += o.x; sacc[nt][1] += o.y; sacc[nt][2] += o.z; sacc[nt][3] += o.w;
                if (keyA >= kc) sacc[nt][0] = sacc[nt][1] = -INFINITY;
                if (keyB >= kc) sacc[nt][2] = sacc[nt][3] = -INFINITY;
                const float m0 = row_m[8 * nt + 2 * c], m1 = row_m[8 * nt + 2 * c + 1];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float m = (q & 1) ? m1 : m0, sv = sacc[nt][q];
                    raise |= (sv > m + kRaise);
                    e[nt][q] = (sv == -INFINITY || m == -INFINITY) ? 0.f : __expf(fminf(sv - m, 2.f * kRaise));
                }
                ps[(8 * nt + 2 * c) * PS + keyA] = __float2half_rn(e[nt][0]);
                ps[(8 * nt + 2 * c + 1) * PS + keyA] = __float2half_rn(e[nt][1]);
                ps[(8 * nt + 2 * c) * PS + keyB] = __float2half_rn(e[nt][2]);
                ps[(8 * nt + 2 * c + 1) * PS + keyB] = __float2half_rn(e[nt][3]);
            }
        }
        if (__syncthreads_or(raise)) {
            // a score passed the reference by more than kRaise: raise it to the running maximum, rescale, redo P
            if (kh == 0) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    float x0 = fmaxf(sacc[nt][0], sacc[nt][2]), x1 = fmaxf(sacc[nt][1], sacc[nt][3]);
#pragma unroll
                    for (int sh = 4; sh < 32; sh <<= 1) {
                        x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, sh));
                        x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, sh));
                    }
                    if (g == 0) { wmax[mt * NH + 8 * nt + 2 * c] = x0; wmax[mt * NH + 8 * nt + 2 * c + 1] = x1; }
                }
            }
            __syncthreads();
            float mnew[NT][2], alpha[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int hh = 8 * nt + 2 * c + q;
                    const float old = row_m[hh];
                    float mx = old;
#pragma unroll
                    for (int w = 0; w < 4; ++w) mx = fmaxf(mx, wmax[w * NH + hh]);
                    mnew[nt][q] = mx;
                    alpha[nt][q] = (old == -INFINITY) ? 0.f : __expf(old - mx);
                }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    oacc[i][nt][0] *= alpha[nt][0]; oacc[i][nt][1] *= alpha[nt][1];
                    oacc[i][nt][2] *= alpha[nt][0]; oacc[i][nt][3] *= alpha[nt][1];
                }
            if (kh == 0) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    lsum[nt][0] *= alpha[nt][0]; lsum[nt][1] *= alpha[nt][1];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float m = mnew[nt][q & 1], sv = sacc[nt][q];
                        e[nt][q] = (sv == -INFINITY) ? 0.f : __expf(sv - m);
                    }
                    ps[(8 * nt + 2 * c) * PS + keyA] = __float2half_rn(e[nt][0]);
                    ps[(8 * nt + 2 * c + 1) * PS + keyA] = __float2half_rn(e[nt][1]);
                    ps[(8 * nt + 2 * c) * PS + keyB] = __float2half_rn(e[nt][2]);
                    ps[(8 * nt + 2 * c + 1) * PS + keyB] = __float2half_rn(e[nt][3]);
                }
            }
            __syncthreads();                                  // P is final; every thread has read the old reference
            if (warp == 0 && g == 0) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) { row_m[8 * nt + 2 * c] = mnew[nt][0]; row_m[8 * nt + 2 * c + 1] = mnew[nt][1]; }
            }
        }
        if (kh == 0) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) { lsum[nt][0] += e[nt][0] + e[nt][2]; lsum[nt][1] += e[nt][1] + e[nt][3]; }
        }
        // ---- O^T += V^T P' : warp w -> dims [64 w, 64 w + 64), P' = P x the keys' scale of this warp's group ----
#pragma unroll
        for (int k0 = 0; k0 < KC; k0 += 16) {
            const __half2 f0 = __floats2half2_rn(sks[(k0 + 2 * c) * NG + grp_w], sks[(k0 + 2 * c + 1) * NG + grp_w]);
            const __half2 f1 = __floats2half2_rn(sks[(k0 + 2 * c + 8) * NG + grp_w], sks[(k0 + 2 * c + 9) * NG + grp_w]);
            uint32_t b[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const __half* pr = ps + (8 * nt + g) * PS + k0 + 2 * c;
                __half2 v0 = __hmul2(*reinterpret_cast<const __half2*>(pr), f0), v1 = __hmul2(*reinterpret_cast<const __half2*>(pr + 8), f1);
                b[nt][0] = *reinterpret_cast<uint32_t*>(&v0);
                b[nt][1] = *reinterpret_cast<uint32_t*>(&v1);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t a[4];
                ldmatrix_x4_trans(a, vrow0 + k0 * DP + 16 * i);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma16816(oacc[i][nt], a, b[nt][0], b[nt][1]);
            }
        }
    }
    // ---- normalise and write the partial ----
    __syncthreads();
    if (kh == 0) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float x0 = lsum[nt][0], x1 = lsum[nt][1];
#pragma unroll
            for (int sh = 4; sh < 32; sh <<= 1) {
                x0 += __shfl_xor_sync(0xffffffffu, x0, sh);
                x1 += __shfl_xor_sync(0xffffffffu, x1, sh);
            }
            if (g == 0) { wl[mt * NH + 8 * nt + 2 * c] = x0; wl[mt * NH + 8 * nt + 2 * c + 1] = x1; }
        }
    }
    __syncthreads();
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int hA = 8 * nt + 2 * c, hB = hA + 1;
        const float lA = wl[hA] + wl[NH + hA] + wl[2 * NH + hA] + wl[3 * NH + hA];
        const float lB = wl[hB] + wl[NH + hB] + wl[2 * NH + hB] + wl[3 * NH + hB];
        const float iA = lA > 0.f ? 1.f / lA : 0.f, iB = lB > 0.f ? 1.f / lB : 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int d = warp * 64 + 16 * i + g;
            if (p.o_final != nullptr) {                       // one split: this is the result, no combine pass
                if (hA < nh) {
                    bf16* o = p.o_final + ((size_t)t * p.h + h0 + hA) * R + d;
                    o[0] = __float2bfloat16(oacc[i][nt][0] * iA); o[8] = __float2bfloat16(oacc[i][nt][2] * iA);
                }
                if (hB < nh) {
                    bf16* o = p.o_final + ((size_t)t * p.h + h0 + hB) * R + d;
                    o[0] = __float2bfloat16(oacc[i][nt][1] * iB); o[8] = __float2bfloat16(oacc[i][nt][3] * iB);
                }
                continue;
            }
            if (hA < nh) {
                float* o = p.o_part + (((size_t)t * p.h + h0 + hA) * p.splits + split) * R + d;
                o[0] = oacc[i][nt][0] * iA; o[8] = oacc[i][nt][2] * iA;
            }
            if (hB < nh) {
                float* o = p.o_part + (((size_t)t * p.h + h0 + hB) * p.splits + split) * R + d;
                o[0] = oacc[i][nt][1] * iB; o[8] = oacc[i][nt][3] * iB;
            }
        }
    }
    if (tid < nh) {
        const float l = wl[tid] + wl[NH + tid] + wl[2 * NH + tid] + wl[3 * NH + tid];
        const float lse = l > 0.f ? row_m[tid] + logf(l) : -INFINITY;
        if (p.o_final != nullptr) {
            if (p.lse_final != nullptr) p.lse_final[(size_t)t * p.h + h0 + tid] = lse;
        } else {
            p.lse_part[((size_t)t * p.h + h0 + tid) * p.splits + split] = lse;
        }
    }
}

template <int NT>
int launch_transposed(const Params& p, int T, cudaStream_t s) {
    using namespace tk;
    constexpr int NH = 8 * NT;
    const size_t smem = (size_t)(NH * DP + KC * DP + NH * PS) * sizeof(__half) + (size_t)(KC * NG) * sizeof(float) +
                        (size_t)(4 * NT * 32) * sizeof(float4) + (size_t)(9 * NH + 2 * KC) * sizeof(float);
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(sparse_mla_mma_t_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        attr = true;
    }
    dim3 grid(p.splits, (p.h + NH - 1) / NH, T);
    sl_launch(sparse_mla_mma_t_kernel<NT>, grid, 256, smem, s, p);
    return (int)cudaGetLastError();
}

// the transposed kernel is compiled for the 656-byte row (512 latent values in groups of 128, 64 rope values)
bool transposed_ok(const Params& p) { return p.R == tk::R && p.group == tk::GS && p.Dr == tk::DR; }

}  // namespace

// Same contract as sl_sparse_mla_split (csrc/sparse_mla.cu).  Needs R % 64 == 0, (R + Dr) % 16 == 0,
// R <= 512, Dr % 2 == 0, group % 4 == 0.  Returns -1 when the shape is not supported.
SL_API int sl_sparse_mla_split_mma(const void* params, int T, cudaStream_t s) {
    const Params* p = static_cast<const Params*>(params);
    if (T == 0) return 0;
    if (p->R % 64 != 0 || p->R > 512 || (p->R + p->Dr) % 16 != 0 || p->Dr % 2 != 0 || p->group % 4 != 0) return -1;
    if (g_transposed_enabled && transposed_ok(*p)) {
        if (p->o_final != nullptr && p->splits != 1) return -1;
        {
            const int r = sparse_mla_tcgen05(p, T, s);           // -2: not a launch it covers
            if (r != -2) return r;
        }
        return p->h <= 8 ? launch_transposed<1>(*p, T, s) : launch_transposed<2>(*p, T, s);
    }
    if (p->o_final != nullptr) return -1;                     // only the keys-on-M kernel writes the final output itself
    const int DP = p->R + p->Dr + 8;
    const size_t smem = (size_t)(HB * DP + KC * DP + HB * 72) * sizeof(__half) + (size_t)(8 * HB * 2 + 3 * HB + 2 * KC) * sizeof(float);
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(sparse_mla_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        attr = true;
    }
    if (smem > 160 * 1024) return -1;
    dim3 grid(p->splits, (p->h + HB - 1) / HB, T);
    sl_launch(sparse_mla_mma_kernel, grid, 256, smem, s, *p);
    return (int)cudaGetLastError();
}

// 0 selects the heads-on-M kernel for every shape (comparison runs); default 1.
SL_API void sl_sparse_mla_set_transposed(int on) { g_transposed_enabled = on != 0; }

// 1 when a launch with these row parameters and one split may be given `o_final` (the keys-on-M kernel takes it).
SL_API int sl_sparse_mla_direct_ok(int R, int group, int Dr) {
    Params p{};
    p.R = R; p.group = group; p.Dr = Dr;
    return (g_transposed_enabled && transposed_ok(p)) ? 1 : 0;
}
