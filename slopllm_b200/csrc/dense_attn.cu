// Dense grouped-query attention over a paged bf16 KV cache (Qwen3 / Qwen3.5 full-attention layers).
//
//  * qk_norm_rope_kernel: per-head RMSNorm + rotary (rotate-half over the first rope_dim dims) of the
//    q and k projections; k and v rows are written straight into their cache slots (the reference runs
//    `fused_norm_rope` + `kv_cache_write` as separate kernels, `csrc/glm_ops.cu`).
//  * paged_attn_prefill_kernel: FlashAttention-2 style, 64 queries x 1 head per CTA on `mma.sync.m16n8k16`
//    bf16 with fp32 accumulation; each warp owns 16 query rows end to end (scores, online softmax and P
//    stay in registers), K/V tiles of 64 keys are gathered from the pages into shared memory.
//  * paged_attn_decode_kernel: split-KV flash decoding for one query token per sequence; one CTA per
//    (token, kv head, split) serves the whole group of query heads, so K/V are read once per group.
//    Partials are merged by `sl_mla_combine`.
// The reference uses FlashInfer's paged prefill / decode for these (`csrc/glm_flash.cu:1-700`).
#include "common.cuh"

namespace {

struct NormRopeParams {
    const bf16* q; int ldq;          // [T, n_heads * q_stride]; head h at h * q_stride (q_stride >= hd: gate packed after q)
    const bf16* k; int ldk;          // [T, n_kv * hd]
    const bf16* v; int ldv;          // [T, n_kv * hd]
    const bf16* q_norm_w;            // [hd] or null
    const bf16* k_norm_w;            // [hd] or null
    const int* positions;            // [T]
    const int* batch_idx;            // [T]
    const int* page_table; int pt_stride, page_size;
    int n_heads, n_kv, hd, q_stride, rope_dim;
    float eps, theta;
    bf16* q_out;                     // [T, n_heads, hd]
    bf16* k_cache;                   // [slots, n_kv, hd]
    bf16* v_cache;
};

// grid (T, n_heads + n_kv); one warp per (token, head) row, lane l holds dims l, l + 32, ...
__global__ void qk_norm_rope_kernel(NormRopeParams p) {
    pdl_grid_sync();
    const int t = blockIdx.x, hh = blockIdx.y, lane = threadIdx.x;
    const bool is_q = hh < p.n_heads;
    const int h = is_q ? hh : hh - p.n_heads;
    const bf16* src = is_q ? p.q + (size_t)t * p.ldq + (size_t)h * p.q_stride : p.k + (size_t)t * p.ldk + (size_t)h * p.hd;
    const bf16* w = is_q ? p.q_norm_w : p.k_norm_w;
    const int pos = p.positions[t];
    const int page = p.page_table[(size_t)p.batch_idx[t] * p.pt_stride + pos / p.page_size];
    const size_t slot = (size_t)page * p.page_size + pos % p.page_size;
    // each lane holds dims lane, lane + 32, ...; up to 8 values (hd <= 256)
    float v[8];
    float ss = 0.f;
    const int per = (p.hd + 31) / 32;
    for (int i = 0; i < per; ++i) {
        const int d = lane + i * 32;
        v[i] = d < p.hd ? __bfloat162float(src[d]) : 0.f;
        ss += v[i] * v[i];
    }
    if (w != nullptr) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)p.hd + p.eps);
        for (int i = 0; i < per; ++i) {
            const int d = lane + i * 32;
            if (d < p.hd) v[i] = __bfloat162float(__float2bfloat16(v[i] * inv * __bfloat162float(w[d])));
        }
    }
    // rotate-half: pairs (d, d + rope_dim/2) for d < rope_dim/2; the partner is fetched through shared memory
    __shared__ float sv[256];
    for (int i = 0; i < per; ++i) {
        const int d = lane + i * 32;
        if (d < p.hd) sv[d] = v[i];
    }
    __syncwarp();
    const int half = p.rope_dim / 2;
    float outv[8];
    for (int i = 0; i < per; ++i) {
        const int d = lane + i * 32;
        outv[i] = v[i];
        if (d < p.rope_dim) {
            const int fi = d < half ? d : d - half;
            const float inv_freq = 1.0f / powf(p.theta, (float)(2 * fi) / (float)p.rope_dim);
            float sn, cs;
            sincosf((float)pos * inv_freq, &sn, &cs);
            const float partner = sv[d < half ? d + half : d - half];
            outv[i] = d < half ? v[i] * cs - partner * sn : v[i] * cs + partner * sn;
        }
    }
    bf16* dst = is_q ? p.q_out + ((size_t)t * p.n_heads + h) * p.hd : p.k_cache + (slot * p.n_kv + h) * p.hd;
    for (int i = 0; i < per; ++i) {
        const int d = lane + i * 32;
        if (d < p.hd) dst[d] = __float2bfloat16(outv[i]);
    }
    if (!is_q) {
        const bf16* vs = p.v + (size_t)t * p.ldv + (size_t)h * p.hd;
        bf16* vd = p.v_cache + (slot * p.n_kv + h) * p.hd;
        for (int d = lane; d < p.hd; d += 32) vd[d] = vs[d];
    }
}

struct AttnParams {
    const bf16* q;                   // [T, n_heads, hd]
    const bf16* k_cache;             // [slots, n_kv, hd]
    const bf16* v_cache;
    const int* positions;            // [T] absolute position of each query (keys 0..pos are visible)
    const int* batch_idx;            // [T]
    const int* page_table; int pt_stride, page_size;
    const int* qo_indptr;            // [B + 1] (prefill)
    int n_heads, n_kv, hd;
    float sm_scale;
    bf16* out;                       // prefill: [T, n_heads, hd]
    float* o_part; float* lse_part;  // decode: [T, n_heads, splits, hd], [T, n_heads, splits]
    int splits;
};

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x2(uint32_t& r0, uint32_t& r1, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(a));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t& r0, uint32_t& r1, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(a));
}

constexpr int QT = 64;      // queries per CTA (4 warps x 16)
constexpr int KT = 64;      // keys per tile

// grid (ceil(max_q / 64), n_heads, B); block 128.  HD in {64, 128}.
template <int HD>
__global__ void __launch_bounds__(128) paged_attn_prefill_kernel(AttnParams p) {
    pdl_grid_sync();
    constexpr int DP = HD + 8;                       // padded row (16-byte aligned, bank-skewed)
    extern __shared__ __align__(16) unsigned char smraw[];
    bf16* qs = reinterpret_cast<bf16*>(smraw);       // [64][DP]
    bf16* ks = qs + QT * DP;                         // [64][DP]
    bf16* vs = ks + KT * DP;                         // [64][DP]
    const int seq = blockIdx.z, hq = blockIdx.y, hkv = hq / (p.n_heads / p.n_kv);
    const int t_begin = p.qo_indptr[seq], t_end = p.qo_indptr[seq + 1];
    const int q0 = t_begin + blockIdx.x * QT;
    if (q0 >= t_end) return;
    const int nq = min(QT, t_end - q0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, c = lane & 3;
    const int* pt = p.page_table + (size_t)p.batch_idx[t_begin] * p.pt_stride;

    // Q tile (rows beyond nq are zero)
    for (int i = tid; i < QT * (HD / 8); i += blockDim.x) {
        const int r = i / (HD / 8), ch = i % (HD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nq) v = *reinterpret_cast<const uint4*>(p.q + ((size_t)(q0 + r) * p.n_heads + hq) * HD + ch * 8);
        *reinterpret_cast<uint4*>(qs + r * DP + ch * 8) = v;
    }
    // positions of this warp's two rows per lane (rows g and g + 8 of the warp tile)
    const int r0 = warp * 16 + g, r1 = r0 + 8;
    const int pos0 = r0 < nq ? p.positions[q0 + r0] : -1, pos1 = r1 < nq ? p.positions[q0 + r1] : -1;
    // last visible key over the CTA: positions ascend within a sequence
    const int max_pos = p.positions[q0 + nq - 1];

    float oacc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const float scale_log2 = p.sm_scale * 1.4426950408889634f;

    for (int k0 = 0; k0 <= max_pos; k0 += KT) {
        __syncthreads();
        // gather K/V tile rows k0 .. k0+63 (rows beyond max_pos are zero)
        for (int i = tid; i < KT * (HD / 8); i += blockDim.x) {
            const int r = i / (HD / 8), ch = i % (HD / 8), kp = k0 + r;
            uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
            if (kp <= max_pos) {
                const size_t slot = (size_t)pt[kp / p.page_size] * p.page_size + kp % p.page_size;
                const size_t off = (slot * p.n_kv + hkv) * HD + ch * 8;
                kv = ldg_nc_16(p.k_cache + off);
                vv = ldg_nc_16(p.v_cache + off);
            }
            *reinterpret_cast<uint4*>(ks + r * DP + ch * 8) = kv;
            *reinterpret_cast<uint4*>(vs + r * DP + ch * 8) = vv;
        }
        __syncthreads();
        // S = Q K^T for this warp's 16 rows x 64 keys
        float s[KT / 8][4];
#pragma unroll
        for (int n = 0; n < KT / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < HD; kk += 16) {
            uint32_t a[4];
            ldsm_x4(a, qs + (warp * 16 + (lane & 15)) * DP + kk + (lane >> 4) * 8);
#pragma unroll
            for (int n = 0; n < KT / 8; ++n) {
                uint32_t b0, b1;
                ldsm_x2(b0, b1, ks + (n * 8 + (lane & 7)) * DP + kk + ((lane >> 3) & 1) * 8);
                mma_bf16_16816(s[n], a, b0, b1);
            }
        }
        // causal mask + online softmax (log2 domain)
        float mx0 = m0, mx1 = m1;
#pragma unroll
        for (int n = 0; n < KT / 8; ++n) {
            const int key = k0 + n * 8 + 2 * c;
            s[n][0] = key <= pos0 ? s[n][0] * scale_log2 : -INFINITY;
            s[n][1] = key + 1 <= pos0 ? s[n][1] * scale_log2 : -INFINITY;
            s[n][2] = key <= pos1 ? s[n][2] * scale_log2 : -INFINITY;
            s[n][3] = key + 1 <= pos1 ? s[n][3] * scale_log2 : -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
            mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float a0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - mx0), a1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - mx1);
        m0 = mx0; m1 = mx1;
        float sum0 = 0.f, sum1 = 0.f;
        uint32_t pa[KT / 16][4];                     // P as bf16 A fragments (k = keys)
#pragma unroll
        for (int n = 0; n < KT / 8; ++n) {
            const float e0 = (s[n][0] == -INFINITY) ? 0.f : exp2f(s[n][0] - m0), e1 = (s[n][1] == -INFINITY) ? 0.f : exp2f(s[n][1] - m0);
            const float e2 = (s[n][2] == -INFINITY) ? 0.f : exp2f(s[n][2] - m1), e3 = (s[n][3] == -INFINITY) ? 0.f : exp2f(s[n][3] - m1);
            sum0 += e0 + e1; sum1 += e2 + e3;
            // accumulator tile n covers keys n*8..n*8+7: A fragment j = n/2, registers {0,1} for even n, {2,3} for odd n
            pa[n >> 1][(n & 1) * 2 + 0] = f2_to_bf162(e0, e1);
            pa[n >> 1][(n & 1) * 2 + 1] = f2_to_bf162(e2, e3);
        }
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
        l0 = l0 * a0 + sum0; l1 = l1 * a1 + sum1;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) { oacc[i][0] *= a0; oacc[i][1] *= a0; oacc[i][2] *= a1; oacc[i][3] *= a1; }
        // O += P V
#pragma unroll
        for (int j = 0; j < KT / 16; ++j) {
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                uint32_t b0, b1;
                ldsm_x2_trans(b0, b1, vs + (j * 16 + (lane & 15)) * DP + i * 8);
                mma_bf16_16816(oacc[i], pa[j], b0, b1);
            }
        }
    }
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        const int d = i * 8 + 2 * c;
        if (r0 < nq) *reinterpret_cast<uint32_t*>(p.out + ((size_t)(q0 + r0) * p.n_heads + hq) * HD + d) = f2_to_bf162(oacc[i][0] * i0, oacc[i][1] * i0);
        if (r1 < nq) *reinterpret_cast<uint32_t*>(p.out + ((size_t)(q0 + r1) * p.n_heads + hq) * HD + d) = f2_to_bf162(oacc[i][2] * i1, oacc[i][3] * i1);
    }
}

// grid (splits, n_kv, T); block 128 = 4 warps.  A warp takes chunks of 32 keys: lane-per-key scores for each of the
// G query heads of the group (q in shared memory), then lane-per-dims accumulation of P V.  G <= 16, hd <= 256.
template <int G, int DPL>
__global__ void __launch_bounds__(128) paged_attn_decode_kernel(AttnParams p) {
    pdl_grid_sync();
    extern __shared__ float dsm[];
    const int hd = p.hd;
    float* qsh = dsm;                                 // [G][hd] (pre-scaled)
    float* psh = qsh + G * hd;                        // [4 warps][G][32]
    float* osh = psh + 4 * G * 32;                    // [4 warps][G][hd] partial outputs
    float* msh = osh + 4 * G * hd;                    // [4 warps][G] max, then [4][G] sum
    const int split = blockIdx.x, hkv = blockIdx.y, t = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pos = p.positions[t], L = pos + 1;
    const int per = (L + p.splits - 1) / p.splits;
    const int kb = min(L, split * per), ke = min(L, kb + per);
    const int* pt = p.page_table + (size_t)p.batch_idx[t] * p.pt_stride;
    for (int i = tid; i < G * hd; i += blockDim.x)
        qsh[i] = __bfloat162float(p.q[((size_t)t * p.n_heads + hkv * G + i / hd) * hd + i % hd]) * p.sm_scale;
    __syncthreads();
    constexpr int dpl = DPL;                          // dims per lane
    float m[G], l[G], o[G][DPL];
#pragma unroll
    for (int gq = 0; gq < G; ++gq) {
        m[gq] = -INFINITY; l[gq] = 0.f;
#pragma unroll
        for (int i = 0; i < dpl; ++i) o[gq][i] = 0.f;
    }
    for (int c0 = kb + warp * 32; c0 < ke; c0 += 4 * 32) {
        const int key = c0 + lane;
        const bool valid = key < ke;
        size_t off = 0;
        if (valid) off = (((size_t)pt[key / p.page_size] * p.page_size + key % p.page_size) * p.n_kv + hkv) * hd;
        // scores
        float sc[G];
#pragma unroll
        for (int gq = 0; gq < G; ++gq) sc[gq] = 0.f;
        if (valid) {
            for (int d = 0; d < hd; d += 8) {
                const uint4 kv = ldg_nc_16(p.k_cache + off + d);
                const float2 k0 = bf162_to_f2(kv.x), k1 = bf162_to_f2(kv.y), k2 = bf162_to_f2(kv.z), k3 = bf162_to_f2(kv.w);
#pragma unroll
                for (int gq = 0; gq < G; ++gq) {
                    const float* qv = qsh + gq * hd + d;
                    sc[gq] += k0.x * qv[0] + k0.y * qv[1] + k1.x * qv[2] + k1.y * qv[3] + k2.x * qv[4] + k2.y * qv[5] + k3.x * qv[6] + k3.y * qv[7];
                }
            }
        }
#pragma unroll
        for (int gq = 0; gq < G; ++gq) {
            const float s = valid ? sc[gq] : -INFINITY;
            const float mx = fmaxf(m[gq], warp_max(s));
            const float alpha = (m[gq] == -INFINITY) ? 0.f : __expf(m[gq] - mx);
            const float e = valid ? __expf(s - mx) : 0.f;
            l[gq] = l[gq] * alpha + warp_sum(e);
            m[gq] = mx;
            psh[(warp * G + gq) * 32 + lane] = e;
#pragma unroll
            for (int i = 0; i < dpl; ++i) o[gq][i] *= alpha;
        }
        __syncwarp();
        // P V: lane owns dims lane*dpl .. (contiguous so that a V row is read with wide loads)
        const int nk = min(32, ke - c0);
        for (int kk = 0; kk < nk; ++kk) {
            const int key2 = c0 + kk;
            const size_t off2 = (((size_t)pt[key2 / p.page_size] * p.page_size + key2 % p.page_size) * p.n_kv + hkv) * hd;
            float vv[DPL];
#pragma unroll
            for (int i = 0; i < dpl; ++i) {
                const int d = lane * dpl + i;
                vv[i] = d < hd ? __bfloat162float(p.v_cache[off2 + d]) : 0.f;
            }
#pragma unroll
            for (int gq = 0; gq < G; ++gq) {
                const float pv = psh[(warp * G + gq) * 32 + kk];
#pragma unroll
                for (int i = 0; i < dpl; ++i) o[gq][i] += pv * vv[i];
            }
        }
        __syncwarp();
    }
    // merge the 4 warps
#pragma unroll
    for (int gq = 0; gq < G; ++gq) {
        if (lane == 0) { msh[warp * G + gq] = m[gq]; msh[4 * G + warp * G + gq] = l[gq]; }
#pragma unroll
        for (int i = 0; i < dpl; ++i) {
            const int d = lane * dpl + i;
            if (d < hd) osh[(warp * G + gq) * hd + d] = o[gq][i];
        }
    }
    __syncthreads();
    for (int i = tid; i < G * hd; i += blockDim.x) {
        const int gq = i / hd, d = i % hd;
        float mx = -INFINITY;
        for (int w = 0; w < 4; ++w) mx = fmaxf(mx, msh[w * G + gq]);
        float den = 0.f, acc = 0.f;
        for (int w = 0; w < 4; ++w) {
            const float mw = msh[w * G + gq];
            const float f = (mw == -INFINITY) ? 0.f : __expf(mw - mx);
            den += f * msh[4 * G + w * G + gq];
            acc += f * osh[(w * G + gq) * hd + d];
        }
        const int hq = hkv * G + gq;
        p.o_part[(((size_t)t * p.n_heads + hq) * p.splits + split) * hd + d] = den > 0.f ? acc / den : 0.f;
        if (d == 0) p.lse_part[((size_t)t * p.n_heads + hq) * p.splits + split] = den > 0.f ? mx + logf(den) : -INFINITY;
    }
}

}  // namespace

SL_API int sl_qk_norm_rope_cache(const NormRopeParams* p, int T, cudaStream_t s) {
    if (T == 0) return 0;
    if (p->hd > 256 || p->rope_dim > p->hd || p->rope_dim % 2 != 0) return -1;
    sl_launch(qk_norm_rope_kernel, dim3(T, p->n_heads + p->n_kv), 32, 0, s, *p);
    return SL_LAUNCH_CHECK();
}

// Causal attention of B sequences' query ranges over their cached keys 0..position.  hd in {64, 128}.
SL_API int sl_paged_attn_prefill(const AttnParams* p, int B, int max_q, cudaStream_t s) {
    if (B == 0 || max_q == 0) return 0;
    if (p->n_heads % p->n_kv != 0) return -1;
    dim3 grid((max_q + QT - 1) / QT, p->n_heads, B);
    if (p->hd == 128) {
        const size_t smem = (size_t)3 * 64 * (128 + 8) * sizeof(bf16);
        auto kern = paged_attn_prefill_kernel<128>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        sl_launch(kern, grid, 128, smem, s, *p);
    } else if (p->hd == 64) {
        const size_t smem = (size_t)3 * 64 * (64 + 8) * sizeof(bf16);
        sl_launch(paged_attn_prefill_kernel<64>, grid, 128, smem, s, *p);
    } else {
        return -1;
    }
    return SL_LAUNCH_CHECK();
}

template <int G>
static int launch_decode(const AttnParams* p, int T, size_t smem, cudaStream_t s) {
    const int dpl = (p->hd + 31) / 32;
#define SL_DEC(D)                                                                                              \
    {                                                                                                          \
        auto kern = paged_attn_decode_kernel<G, D>;                                                            \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        sl_launch(kern, dim3(p->splits, p->n_kv, T), 128, smem, s, *p);                                        \
    }
    if (dpl <= 2) SL_DEC(2) else if (dpl <= 4) SL_DEC(4) else SL_DEC(8)
#undef SL_DEC
    return SL_LAUNCH_CHECK();
}

// One query token per row t (decode): partial (o, lse) per split, to be merged by sl_mla_combine.
// Query heads per kv head in {1, 2, 4, 8, 16}.
SL_API int sl_paged_attn_decode(const AttnParams* p, int T, cudaStream_t s) {
    if (T == 0) return 0;
    const int G = p->n_heads / p->n_kv;
    if (p->n_heads % p->n_kv != 0 || p->hd > 256 || p->hd % 8 != 0) return -1;
    const size_t smem = (size_t)(G * p->hd + 4 * G * 32 + 4 * G * p->hd + 8 * G) * sizeof(float);
    switch (G) {
        case 1: return launch_decode<1>(p, T, smem, s);
        case 2: return launch_decode<2>(p, T, smem, s);
        case 4: return launch_decode<4>(p, T, smem, s);
        case 8: return launch_decode<8>(p, T, smem, s);
        case 16: return launch_decode<16>(p, T, smem, s);
        default: return -1;
    }
}
