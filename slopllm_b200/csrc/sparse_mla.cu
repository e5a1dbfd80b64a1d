// Sparse MLA attention over gathered packed rows (fp8 latent + per-group scale + bf16 rope),
// split over the selected keys with a log-sum-exp combine, plus the cross-rank merge used by
// context parallelism.
//
// Reference: the vendored sparse-MLA decode/prefill kernels behind `csrc/glm_sparse_mla.cu:34-126`
// (split-K over top-k, mid_out/mid_lse, combine) and `csrc/glm_context_parallel.cu:39-540`.
#include "common.cuh"

struct SparseMlaParams {
    const bf16* q_abs;        // [T, h, R]
    const bf16* q_pe;         // [T, h, Dr]
    const uint8_t* kv_cache;  // [slots, row_bytes]
    const int* slots;         // [T, topk]
    const int* lengths;       // [T]
    int h, R, Dr, group, topk, splits;
    float sm_scale;
    float* o_part;            // [T, h, splits, R]
    float* lse_part;          // [T, h, splits]
    int num_slots;            // rows of kv_cache (0 = unknown: no check)
    int* guard;               // index self-check record (see guard_ok), may be null
};

// grid (splits, head groups of HB, T); block 256.
// Shared: q [HB][DP], k [KC][DP] (dequantised fp32, row pitch DP = R + Dr + 1), p [HB][KC].
template <int HB, int KC>
__global__ void __launch_bounds__(256) sparse_mla_split_kernel(SparseMlaParams p) {
    pdl_grid_sync();
    extern __shared__ float sm[];
    const int D = p.R + p.Dr, DP = D + 1;
    float* qs = sm;                       // HB * DP
    float* ks = qs + HB * DP;             // KC * DP
    float* ps = ks + KC * DP;             // HB * KC
    float* alpha_s = ps + HB * KC;        // HB
    const int split = blockIdx.x, hg = blockIdx.y, t = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int L = p.lengths[t];
    const int per = (L + p.splits - 1) / p.splits;
    const int j_begin = min(L, split * per), j_end = min(L, j_begin + per);
    const int h0 = hg * HB;
    const int nh = min(HB, p.h - h0);
    const int ngroups = p.R / p.group;
    const int row_bytes = p.R + 4 * ngroups + 2 * p.Dr;

    for (int i = tid; i < HB * D; i += blockDim.x) {
        const int hh = i / D, d = i % D;
        float v = 0.f;
        if (hh < nh) {
            v = d < p.R ? __bfloat162float(p.q_abs[((size_t)t * p.h + h0 + hh) * p.R + d])
                        : __bfloat162float(p.q_pe[((size_t)t * p.h + h0 + hh) * p.Dr + (d - p.R)]);
        }
        qs[hh * DP + d] = v * p.sm_scale;
    }
    // running state: warp w owns head w (HB <= 8): m, l ; every thread owns output dims
    float m_run = -INFINITY, l_run = 0.f;
    constexpr int MAXDPT = 4;             // dims per thread (R <= 1024)
    float acc[HB][MAXDPT];
#pragma unroll
    for (int a = 0; a < HB; ++a)
#pragma unroll
        for (int b = 0; b < MAXDPT; ++b) acc[a][b] = 0.f;
    const int* slots = p.slots + (size_t)t * p.topk;

    for (int c0 = j_begin; c0 < j_end; c0 += KC) {
        const int kc = min(KC, j_end - c0);
        __syncthreads();
        // dequantise kc rows into shared memory
        for (int i = tid; i < kc * (row_bytes / 4); i += blockDim.x) {
            const int j = i / (row_bytes / 4), wd = i % (row_bytes / 4);
            int slot_j = slots[c0 + j];
            if (p.num_slots != 0 && !guard_ok(p.guard, 12, slot_j, p.num_slots)) slot_j = 0;
            const uint8_t* row = p.kv_cache + (size_t)slot_j * row_bytes;
            const uint32_t u = *reinterpret_cast<const uint32_t*>(row + wd * 4);
            const int byte = wd * 4;
            if (byte < p.R) {
                const float sc = *reinterpret_cast<const float*>(row + p.R + 4 * (byte / p.group));
                const float2 a = e4m3x2_to_float2((uint16_t)(u & 0xffffu)), b = e4m3x2_to_float2((uint16_t)(u >> 16));
                float* dst = ks + j * DP + byte;
                dst[0] = a.x * sc; dst[1] = a.y * sc; dst[2] = b.x * sc; dst[3] = b.y * sc;
            } else if (byte >= p.R + 4 * ngroups) {
                const int d = p.R + (byte - p.R - 4 * ngroups) / 2;
                const float2 f = bf162_to_f2(u);
                ks[j * DP + d] = f.x; ks[j * DP + d + 1] = f.y;
            }
        }
        __syncthreads();
        // scores: warp = head, lanes over keys
        if (warp < HB) {
            float mx = -INFINITY;
            float sv[(KC + 31) / 32];
#pragma unroll
            for (int r = 0; r < (KC + 31) / 32; ++r) {
                const int j = lane + r * 32;
                float s = -INFINITY;
                if (j < kc && warp < nh) {
                    s = 0.f;
                    const float* qh = qs + warp * DP;
                    const float* kj = ks + j * DP;
                    for (int d = 0; d < D; ++d) s += qh[d] * kj[d];
                }
                sv[r] = s;
                mx = fmaxf(mx, s);
            }
            mx = warp_max(mx);
            const float m_new = fmaxf(m_run, mx);
            const float alpha = (m_run == -INFINITY) ? 0.f : __expf(m_run - m_new);
            float sum = 0.f;
#pragma unroll
            for (int r = 0; r < (KC + 31) / 32; ++r) {
                const int j = lane + r * 32;
                const float e = (sv[r] == -INFINITY) ? 0.f : __expf(sv[r] - m_new);
                if (j < KC) ps[warp * KC + j] = e;
                sum += e;
            }
            sum = warp_sum(sum);
            l_run = l_run * alpha + sum;
            m_run = m_new;
            if (lane == 0) alpha_s[warp] = alpha;
        }
        __syncthreads();
        // o += p . ckv : thread owns dims tid, tid+256, ...
#pragma unroll
        for (int a = 0; a < HB; ++a) {
            const float al = alpha_s[a];
#pragma unroll
            for (int b = 0; b < MAXDPT; ++b) acc[a][b] *= al;
        }
        for (int j = 0; j < kc; ++j) {
            float v[MAXDPT];
#pragma unroll
            for (int b = 0; b < MAXDPT; ++b) {
                const int d = tid + b * 256;
                v[b] = d < p.R ? ks[j * DP + d] : 0.f;
            }
#pragma unroll
            for (int a = 0; a < HB; ++a) {
                const float pj = ps[a * KC + j];
#pragma unroll
                for (int b = 0; b < MAXDPT; ++b) acc[a][b] += pj * v[b];
            }
        }
    }
    __syncthreads();
    if (warp < HB && lane == 0) { ps[warp] = l_run; ps[HB + warp] = m_run; }
    __syncthreads();
#pragma unroll
    for (int a = 0; a < HB; ++a) {
        if (a >= nh) break;
        const float l = ps[a], m = ps[HB + a];
        const float inv = l > 0.f ? 1.f / l : 0.f;
        float* o = p.o_part + (((size_t)t * p.h + h0 + a) * p.splits + split) * p.R;
#pragma unroll
        for (int b = 0; b < MAXDPT; ++b) {
            const int d = tid + b * 256;
            if (d < p.R) o[d] = acc[a][b] * inv;
        }
        if (tid == 0) p.lse_part[((size_t)t * p.h + h0 + a) * p.splits + split] = l > 0.f ? m + logf(l) : -INFINITY;
    }
}

SL_API int sl_sparse_mla_split(const SparseMlaParams* p, int T, cudaStream_t s) {
    if (T == 0) return 0;
    if (p->R > 1024 || p->R % 4 != 0 || p->Dr % 2 != 0 || p->group % 4 != 0) return -1;
    constexpr int HB = 8, KC = 32;
    const int DP = p->R + p->Dr + 1;
    const size_t smem = (size_t)(HB * DP + KC * DP + HB * KC + HB) * sizeof(float);
    auto kern = sparse_mla_split_kernel<HB, KC>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dim3 grid(p->splits, (p->h + HB - 1) / HB, T);
    sl_launch(kern, grid, 256, smem, s, *p);
    return SL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Combine `n_part` partial results per (token, head): o = sum_i w_i o_i / sum_i w_i,
// w_i = exp(lse_i - max), lse = max + log(sum w).  Partials may live in several buffers
// (context-parallel ranks): element (tok, head, part) of buffer b is at
// o_ptrs[b] + ((tok*h + head)*parts_per_buf + part)*R.
struct CombineParams {
    const float* o_ptrs[8];
    const float* lse_ptrs[8];
    int n_buf, parts_per_buf, h, R;
    int head_begin, head_count;          // heads written (CP: this rank's slice)
    void* o_out;                         // [T, head_count, R] bf16 (or fp32 when out_f32)
    float* lse_out;                      // [T, head_count] or null
    int out_f32;
    // double-buffered staging (context-parallel merge): when parity_epoch is set, every input pointer is advanced
    // by ((*parity_epoch - 1) & 1) strides; reading the parity on the device keeps a replayed CUDA graph valid
    const uint32_t* parity_epoch;
    long long parity_o_stride, parity_lse_stride;     // in floats
};

__global__ void __launch_bounds__(128) mla_combine_kernel(CombineParams p) {
    pdl_grid_sync();
    const int t = blockIdx.y, hh = blockIdx.x, head = p.head_begin + hh;
    __shared__ float wsh[8 * 64];
    __shared__ float scratch[33];
    const int np = p.n_buf * p.parts_per_buf;
    const size_t th = (size_t)t * p.h + head;
    const size_t par = p.parity_epoch != nullptr ? ((*p.parity_epoch - 1u) & 1u) : 0u;
    const size_t po = par * (size_t)p.parity_o_stride, pl = par * (size_t)p.parity_lse_stride;
    // weights: one partial per thread (np <= 512 -> up to 4 per thread)
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < np; i += blockDim.x) {
        const int b = i / p.parts_per_buf, q = i % p.parts_per_buf;
        const float l = p.lse_ptrs[b][pl + th * p.parts_per_buf + q];
        wsh[i] = l;
        mx = fmaxf(mx, l);
    }
    mx = block_max(mx, scratch);
    float den = 0.f;
    for (int i = threadIdx.x; i < np; i += blockDim.x) {
        const float l = wsh[i];
        const float w = (l == -INFINITY) ? 0.f : __expf(l - mx);
        wsh[i] = w;
        den += w;
    }
    den = block_sum(den, scratch);
    const float inv = den > 0.f ? 1.f / den : 0.f;
    for (int d = threadIdx.x * 4; d < p.R; d += blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        // four independent loads in flight per step; zero-weight partials are finite (written by the split kernel)
        for (int i0 = 0; i0 < np; i0 += 4) {
            float4 v[4];
            float w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = min(i0 + u, np - 1);
                const int b = i / p.parts_per_buf, q = i % p.parts_per_buf;
                w[u] = (i0 + u < np) ? wsh[i] : 0.f;
                v[u] = *reinterpret_cast<const float4*>(p.o_ptrs[b] + po + (th * p.parts_per_buf + q) * p.R + d);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                acc.x += w[u] * v[u].x; acc.y += w[u] * v[u].y; acc.z += w[u] * v[u].z; acc.w += w[u] * v[u].w;
            }
        }
        const size_t oi = ((size_t)t * p.head_count + hh) * p.R + d;
        if (p.out_f32) {
            *reinterpret_cast<float4*>((float*)p.o_out + oi) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        } else {
            uint2 o;
            o.x = f2_to_bf162(acc.x * inv, acc.y * inv);
            o.y = f2_to_bf162(acc.z * inv, acc.w * inv);
            *reinterpret_cast<uint2*>((bf16*)p.o_out + oi) = o;
        }
    }
    if (threadIdx.x == 0 && p.lse_out) p.lse_out[(size_t)t * p.head_count + hh] = den > 0.f ? mx + logf(den) : -INFINITY;
}

SL_API int sl_mla_combine(const CombineParams* p, int T, cudaStream_t s) {
    if (T == 0 || p->head_count == 0) return 0;
    if (p->n_buf * p->parts_per_buf > 8 * 64) return -1;
    sl_launch(mla_combine_kernel, dim3(p->head_count, T), 128, 0, s, *p);
    return SL_LAUNCH_CHECK();
}
