// Normalisation, rotary, cache-row packing, routing top-k and small glue kernels (sm_100a).
//
// Covers what the reference spreads over `csrc/glm_ops.cu` (rmsnorm :210, fused add+rmsnorm
// :358, rotary :1820-1876, layernorm :1029, route_top8 :2343, silu_and_mul :994,
// rotate_input_ids :3308), `csrc/glm_flash.cu:1081-1230` (packed ckv row) and
// `csrc/glm_indexer.cu:303-376,1338` (topk_to_slots, indexer Q quantise), fused along the
// data flow of one decoder layer.
#include "common.cuh"
#include "route.cuh"

int g_sl_pdl_enabled = 1;
unsigned long long g_sl_kernel_launches = 0;
SL_API unsigned long long sl_kernel_launches() { return g_sl_kernel_launches; }
// Turns programmatic dependent launch of the library's kernels on or off (process-wide).
SL_API void sl_set_pdl(int enabled) { g_sl_pdl_enabled = enabled ? 1 : 0; }

// ---------------------------------------------------------------------------------------------
// embedding lookup: out[t, :] = table[ids[t], :]
__global__ void embed_kernel(bf16* __restrict__ out, const int64_t* __restrict__ ids, const bf16* __restrict__ table,
                             int H, int V) {
    pdl_grid_sync();
    const int t = blockIdx.x;
    int64_t id = ids[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);      // never read outside the table
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * H);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)t * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

SL_API int sl_embed(void* out, const void* ids, const void* table, int T, int H, int V, cudaStream_t s) {
    if (T == 0) return 0;
    sl_launch(embed_kernel, T, 256, 0, s, (bf16*)out, (const int64_t*)ids, (const bf16*)table, H, V);
    return SL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// residual' = residual + x (fp32) ; out = rmsnorm(residual') * w (bf16).
// x is bf16 or fp32 (`x_f32`); residual_in may be null (first layer).  H % 4 == 0, H <= 16384.
// One block per token; a thread keeps its (up to 4) float4 chunks in registers between the
// sum-of-squares pass and the scaling pass.
template <bool XF32>
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(bf16* __restrict__ out, float* __restrict__ res_out,
                                                           const void* __restrict__ xin, const float* __restrict__ res_in,
                                                           const bf16* __restrict__ w, int H, float eps, uint4* __restrict__ xp) {
    pdl_grid_sync();
    __shared__ float scratch[33];
    const int t = blockIdx.x, nt = blockDim.x, n4 = H / 4;
    float4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int i = threadIdx.x + q * nt;
        if (i < n4) {
            float4 a;
            if (XF32) {
                a = reinterpret_cast<const float4*>((const float*)xin + (size_t)t * H)[i];
            } else {
                const uint2 u = reinterpret_cast<const uint2*>((const bf16*)xin + (size_t)t * H)[i];
                const float2 lo = bf162_to_f2(u.x), hi = bf162_to_f2(u.y);
                a = make_float4(lo.x, lo.y, hi.x, hi.y);
            }
            if (res_in != nullptr) {
                const float4 r = reinterpret_cast<const float4*>(res_in + (size_t)t * H)[i];
                a.x += r.x; a.y += r.y; a.z += r.z; a.w += r.w;
            }
            v[q] = a;
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int i = threadIdx.x + q * nt;
        if (i < n4) {
            if (res_out != nullptr) reinterpret_cast<float4*>(res_out + (size_t)t * H)[i] = v[q];
            const uint2 wu = reinterpret_cast<const uint2*>(w)[i];
            const float2 w0 = bf162_to_f2(wu.x), w1 = bf162_to_f2(wu.y);
            uint2 o;
            o.x = f2_to_bf162(v[q].x * inv * w0.x, v[q].y * inv * w0.y);
            o.y = f2_to_bf162(v[q].z * inv * w1.x, v[q].w * inv * w1.y);
            reinterpret_cast<uint2*>(out + (size_t)t * H)[i] = o;
            if (xp != nullptr) store_perm4(xp, t, H, i, o.x, o.y);
        }
    }
}

// `xp` (optional): also write the normed row as the permuted f16 copy that the NVFP4 tensor-core kernels consume
// (H % 128 == 0; rows of the copy beyond T are never read for valid outputs).
SL_API int sl_add_rmsnorm(void* out, void* res_out, const void* x, const void* res_in, const void* w, int T, int H,
                          float eps, int x_f32, void* xp, cudaStream_t s) {
    if (T == 0) return 0;
    if (H % 4 != 0 || H > 16384 || (xp != nullptr && H % 128 != 0)) return -1;
    int threads = ((H / 4 + 3) / 4 + 31) / 32 * 32;      // 4 chunks per thread when possible
    if (threads < 128) threads = 128;
    if (threads > 1024) threads = 1024;
    if (x_f32)
        sl_launch(add_rmsnorm_kernel<true>, T, threads, 0, s, (bf16*)out, (float*)res_out, x, (const float*)res_in, (const bf16*)w, H, eps,
                  (uint4*)xp);
    else
        sl_launch(add_rmsnorm_kernel<false>, T, threads, 0, s, (bf16*)out, (float*)res_out, x, (const float*)res_in, (const bf16*)w, H, eps,
                  (uint4*)xp);
    return SL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Rotary helper: rotate pair index i (0 <= i < rope_dim/2) of a vector held in shared memory.
__device__ __forceinline__ void rope_pair(float* v, int i, int rope_dim, int pos, float theta, bool interleave) {
    const float inv_freq = 1.0f / powf(theta, (float)(2 * i) / (float)rope_dim);
    const float ang = (float)pos * inv_freq;
    float sn, cs;
    sincosf(ang, &sn, &cs);
    const int ia = interleave ? 2 * i : i;
    const int ib = interleave ? 2 * i + 1 : i + rope_dim / 2;
    const float a = v[ia], b = v[ib];
    v[ia] = a * cs - b * sn;
    v[ib] = a * sn + b * cs;
}

// Activation that is either bf16 [T, ld] (n_slabs == 0) or a sum of n_slabs fp32 slabs [T, ld] left by a split-K
// GEMM; the sum is rounded to bf16 so both forms give the same value.
__device__ __forceinline__ float load_act(const void* base, int n_slabs, long long slab_stride, size_t idx) {
    if (n_slabs == 0) return __bfloat162float(reinterpret_cast<const bf16*>(base)[idx]);
    float v = 0.f;
    for (int s = 0; s < n_slabs; ++s) v += reinterpret_cast<const float*>(base)[(size_t)s * slab_stride + idx];
    return __bfloat162float(__float2bfloat16(v));
}

struct AttnPreParams {
    const void* qkv;          // [T, ld] bf16, or fp32 slabs (see load_act)
    int ld;
    int q_lora, kv_lora, rope_dim, idx_dim, idx_heads;   // idx_dim == 0: no indexer in this layer
    const bf16 *q_norm_w, *kv_norm_w, *idx_ln_w, *idx_ln_b;
    float eps, theta;
    int rope_interleave, idx_rope_interleave;
    const int* positions;     // [T]
    const int* batch_idx;     // [T]
    const int* page_table;    // [B, pt_stride]
    int pt_stride, page_size, cp_world, cp_rank;
    int kv_group;             // values per fp8 scale
    uint8_t* kv_cache;        // [slots, kv_row_bytes]
    uint8_t* idx_cache;       // [slots, idx_dim + 4]
    bf16* cq_out;             // [T, q_lora]
    float* idx_w_out;         // [T, idx_heads]
    int n_slabs; long long slab_stride;
    int num_slots;            // rows of the caches (0 = unknown: no check)
    int* guard;               // index self-check record (see guard_ok), may be null
};

// grid (T, 3): three independent pieces of work per token run as separate blocks.
//   role 0  c_q = rmsnorm(q_a)
//   role 1  ckv RMSNorm -> fp8 groups; k_pe RoPE; packed cache row write
//   role 2  indexer key LayerNorm -> RoPE -> fp8 (power-of-two scale) row write; indexer head weights
__global__ void attn_pre_kernel(AttnPreParams p) {
    pdl_grid_sync();
    extern __shared__ float sm[];
    __shared__ float scratch[33];
    const int t = blockIdx.x, role = blockIdx.y, tid = threadIdx.x, nt = blockDim.x;
    const size_t row = (size_t)t * p.ld;
    const int pos = p.positions[t];

    if (role == 0) {
        float ss = 0.f;
        for (int i = tid; i < p.q_lora; i += nt) {
            const float v = load_act(p.qkv, p.n_slabs, p.slab_stride, row + i);
            sm[i] = v;
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        const float inv = rsqrtf(ss / (float)p.q_lora + p.eps);
        for (int i = tid; i < p.q_lora; i += nt)
            p.cq_out[(size_t)t * p.q_lora + i] = __float2bfloat16(sm[i] * inv * __bfloat162float(p.q_norm_w[i]));
        return;
    }
    if (role == 2 && p.idx_dim == 0) return;

    // --- where does this token's row live on this rank? ---
    bool owned = true;
    int local = pos;
    if (p.cp_world > 1) {
        owned = (pos % p.cp_world) == p.cp_rank;
        local = pos / p.cp_world;
    }
    if (!guard_ok(p.guard, 41, local / p.page_size, p.pt_stride)) return;     // block-uniform
    const int page = p.page_table[(size_t)p.batch_idx[t] * p.pt_stride + local / p.page_size];
    const size_t slot = (size_t)page * p.page_size + (local % p.page_size);
    if (p.num_slots != 0 && !guard_ok(p.guard, 42, (long long)slot, p.num_slots)) return;
    const size_t kv = row + p.q_lora;

    if (role == 1) {
        // --- ckv = rmsnorm(kv_a[:R]) rounded to bf16, k_pe = rope(kv_a[R:R+Dr]) ---
        float* ckv = sm;                         // [kv_lora]
        float* kpe = sm + p.kv_lora;             // [rope_dim]
        float ss = 0.f;
        for (int i = tid; i < p.kv_lora; i += nt) {
            const float v = load_act(p.qkv, p.n_slabs, p.slab_stride, kv + i);
            ckv[i] = v;
            ss += v * v;
        }
        for (int i = tid; i < p.rope_dim; i += nt) kpe[i] = load_act(p.qkv, p.n_slabs, p.slab_stride, kv + p.kv_lora + i);
        ss = block_sum(ss, scratch);
        const float inv = rsqrtf(ss / (float)p.kv_lora + p.eps);
        for (int i = tid; i < p.kv_lora; i += nt)
            ckv[i] = __bfloat162float(__float2bfloat16(ckv[i] * inv * __bfloat162float(p.kv_norm_w[i])));
        if (tid < p.rope_dim / 2) rope_pair(kpe, tid, p.rope_dim, pos, p.theta, p.rope_interleave != 0);
        __syncthreads();
        if (!owned) return;
        const int ngroups = p.kv_lora / p.kv_group;
        const int row_bytes = p.kv_lora + 4 * ngroups + 2 * p.rope_dim;
        uint8_t* dst = p.kv_cache + slot * row_bytes;
        // one warp per quantisation group
        const int warp = tid >> 5, lane = tid & 31, nw = nt >> 5;
        for (int g = warp; g < ngroups; g += nw) {
            float amax = 0.f;
            for (int i = lane; i < p.kv_group; i += 32) amax = fmaxf(amax, fabsf(ckv[g * p.kv_group + i]));
            amax = warp_max(amax);
            const float scale = fmaxf(amax / 448.f, FLT_MIN);
            if (lane == 0) reinterpret_cast<float*>(dst + p.kv_lora)[g] = scale;
            for (int i = lane; i < p.kv_group; i += 32)
                dst[g * p.kv_group + i] = float_to_e4m3(ckv[g * p.kv_group + i] / scale);
        }
        bf16* dpe = reinterpret_cast<bf16*>(dst + p.kv_lora + 4 * ngroups);
        for (int i = tid; i < p.rope_dim; i += nt) dpe[i] = __float2bfloat16(kpe[i]);
        return;
    }

    // --- role 2: indexer key and head weights ---
    const size_t ik = kv + p.kv_lora + p.rope_dim;
    float* kbuf = sm;
    float s1 = 0.f;
    for (int i = tid; i < p.idx_dim; i += nt) {
        const float v = load_act(p.qkv, p.n_slabs, p.slab_stride, ik + i);
        kbuf[i] = v;
        s1 += v;
    }
    const float mean = block_sum(s1, scratch) / (float)p.idx_dim;
    float s2 = 0.f;
    for (int i = tid; i < p.idx_dim; i += nt) {
        const float d = kbuf[i] - mean;
        s2 += d * d;
    }
    const float var = block_sum(s2, scratch) / (float)p.idx_dim;
    const float rstd = rsqrtf(var + 1e-6f);
    for (int i = tid; i < p.idx_dim; i += nt)
        kbuf[i] = (kbuf[i] - mean) * rstd * __bfloat162float(p.idx_ln_w[i]) + __bfloat162float(p.idx_ln_b[i]);
    __syncthreads();
    if (tid < p.rope_dim / 2) rope_pair(kbuf, tid, p.rope_dim, pos, p.theta, p.idx_rope_interleave != 0);
    __syncthreads();
    float amax = 0.f;
    for (int i = tid; i < p.idx_dim; i += nt) {
        kbuf[i] = __bfloat162float(__float2bfloat16(kbuf[i]));
        amax = fmaxf(amax, fabsf(kbuf[i]));
    }
    amax = block_max(amax, scratch);
    const float scale = pow2_scale_ceil(amax);
    if (owned) {
        uint8_t* dst = p.idx_cache + slot * (size_t)(p.idx_dim + 4);
        for (int i = tid; i < p.idx_dim; i += nt) dst[i] = float_to_e4m3(kbuf[i] / scale);
        if (tid == 0) {
            // the row is idx_dim + 4 bytes: 4-byte aligned because idx_dim % 4 == 0
            *reinterpret_cast<float*>(dst + p.idx_dim) = scale;
        }
    }
    const float hs = rsqrtf((float)p.idx_heads);
    for (int i = tid; i < p.idx_heads; i += nt)
        p.idx_w_out[(size_t)t * p.idx_heads + i] = load_act(p.qkv, p.n_slabs, p.slab_stride, ik + p.idx_dim + i) * hs;
}

SL_API int sl_attn_pre(const AttnPreParams* p, int T, cudaStream_t s) {
    if (T == 0) return 0;
    int n = p->q_lora > p->kv_lora + p->rope_dim ? p->q_lora : p->kv_lora + p->rope_dim;
    if (p->idx_dim > n) n = p->idx_dim;
    sl_launch(attn_pre_kernel, dim3(T, 3), 256, (size_t)n * sizeof(float), s, *p);
    return SL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// After the q_b | indexer wq_b projection.  grid (T, heads_local + idx_heads).
//  MLA head h:    q_pe[t,h,:] = rope(qb[t, h*dqk + Dn : h*dqk + Dn + Dr])
//  indexer head j: rope(first rope_dim of qi[t,j,:]) -> bf16 -> fp8 with power-of-two scale;
//                  w_eff[t,j] = idx_w[t,j] * scale * Di^-0.5
struct QPostParams {
    const void* qb;           // [T, ld] bf16, or fp32 slabs (see load_act)
    int ld, heads, d_nope, rope_dim, idx_heads, idx_dim;
    float theta;
    int rope_interleave, idx_rope_interleave;
    const int* positions;
    const float* idx_w;       // [T, idx_heads]
    bf16* q_pe_out;           // [T, heads, rope_dim]
    uint8_t* q8_out;          // [T, idx_heads, idx_dim]
    float* w_eff_out;         // [T, idx_heads]
    int n_slabs; long long slab_stride;
};

__device__ __forceinline__ void q_post_body(const QPostParams& p, int t, int hh) {
    __shared__ float v[512];
    __shared__ float scratch[33];
    const int tid = threadIdx.x;
    const int pos = p.positions[t];
    const int dqk = p.d_nope + p.rope_dim;
    if (hh < p.heads) {
        const size_t src = (size_t)t * p.ld + (size_t)hh * dqk + p.d_nope;
        for (int i = tid; i < p.rope_dim; i += blockDim.x) v[i] = load_act(p.qb, p.n_slabs, p.slab_stride, src + i);
        __syncthreads();
        if (tid < p.rope_dim / 2) rope_pair(v, tid, p.rope_dim, pos, p.theta, p.rope_interleave != 0);
        __syncthreads();
        bf16* dst = p.q_pe_out + ((size_t)t * p.heads + hh) * p.rope_dim;
        for (int i = tid; i < p.rope_dim; i += blockDim.x) dst[i] = __float2bfloat16(v[i]);
    } else {
        const int j = hh - p.heads;
        const size_t src = (size_t)t * p.ld + (size_t)p.heads * dqk + (size_t)j * p.idx_dim;
        for (int i = tid; i < p.idx_dim; i += blockDim.x) v[i] = load_act(p.qb, p.n_slabs, p.slab_stride, src + i);
        __syncthreads();
        if (tid < p.rope_dim / 2) rope_pair(v, tid, p.rope_dim, pos, p.theta, p.idx_rope_interleave != 0);
        __syncthreads();
        float amax = 0.f;
        for (int i = tid; i < p.idx_dim; i += blockDim.x) {
            v[i] = __bfloat162float(__float2bfloat16(v[i]));
            amax = fmaxf(amax, fabsf(v[i]));
        }
        amax = block_max(amax, scratch);
        const float scale = pow2_scale_ceil(amax);
        uint8_t* dst = p.q8_out + ((size_t)t * p.idx_heads + j) * p.idx_dim;
        for (int i = tid; i < p.idx_dim; i += blockDim.x) dst[i] = float_to_e4m3(v[i] / scale);
        if (tid == 0)
            p.w_eff_out[(size_t)t * p.idx_heads + j] = p.idx_w[(size_t)t * p.idx_heads + j] * scale * rsqrtf((float)p.idx_dim);
    }
}

__global__ void q_post_kernel(QPostParams p) {
    pdl_grid_sync();
    q_post_body(p, blockIdx.x, blockIdx.y);
}

SL_API int sl_q_post(const QPostParams* p, int T, cudaStream_t s) {
    if (T == 0) return 0;
    dim3 grid(T, p->heads + p->idx_heads);
    sl_launch(q_post_kernel, grid, 64, 0, s, *p);
    return SL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Batched vector x matrix: y[t,h,n] = sum_k x[t,h,k] * M[h,k,n]   (absorb: K=Dn,N=R; v_expand: K=R,N=Dv)
// x element (t,h,k) at x[t*xs_t + h*xs_h + k]; y bf16 [T, Hh, N] contiguous.
// grid (Hh, N/32, ceil(T/TT)); block 256 = 8 warps.  A warp reads 8 matrix rows x 32 columns
// per load instruction (8 columns per lane, 16 bytes), four loads in flight; the partial sums
// of a lane's row group meet by shuffle, those of the 8 warps in shared memory.
// `stage(xs)` fills xs[TT][K] (fp32) with the rows t0 .. t0+TT-1 of head h (zero beyond T); when `xp` is given the
// result is also written as f16 in the fragment order of the NVFP4 streaming kernels (rows up to `tpad`).
template <int TT, typename Stage>
__device__ __forceinline__ void bmv_core(bf16* __restrict__ y, uint4* __restrict__ xp, const bf16* __restrict__ M, int T,
                                         int Hh, int K, int N, int h, int n0, int t0, Stage stage) {
    extern __shared__ float xs[];            // [TT][K], then red[8][TT][32]
    float* red = xs + TT * K;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cg = lane & 3, kr = lane >> 2;
    const int n = n0 + cg * 8;
    const bf16* Mp = M + (size_t)h * K * N + n;
    // the first weight loads do not depend on x: issue them before staging x
    uint4 u[4];
    int k = warp * 8 + kr;
#pragma unroll
    for (int q = 0; q < 4; ++q) u[q] = (n < N && k + q * 64 < K) ? ldg_nc_16(Mp + (size_t)(k + q * 64) * N) : make_uint4(0, 0, 0, 0);
    stage(xs);
    __syncthreads();
    float acc[TT][8];
#pragma unroll
    for (int tt = 0; tt < TT; ++tt)
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[tt][c] = 0.f;
    if (n < N) {
        for (; k < K; k += 256) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                if (k + q * 64 < K) {
                    const float2 w0 = bf162_to_f2(u[q].x), w1 = bf162_to_f2(u[q].y), w2 = bf162_to_f2(u[q].z), w3 = bf162_to_f2(u[q].w);
#pragma unroll
                    for (int tt = 0; tt < TT; ++tt) {
                        const float xv = xs[tt * K + k + q * 64];
                        acc[tt][0] += xv * w0.x; acc[tt][1] += xv * w0.y; acc[tt][2] += xv * w1.x; acc[tt][3] += xv * w1.y;
                        acc[tt][4] += xv * w2.x; acc[tt][5] += xv * w2.y; acc[tt][6] += xv * w3.x; acc[tt][7] += xv * w3.y;
                    }
                }
            }
            const int kn = k + 256;
            if (kn < K) {
#pragma unroll
                for (int q = 0; q < 4; ++q) u[q] = (kn + q * 64 < K) ? ldg_nc_16(Mp + (size_t)(kn + q * 64) * N) : make_uint4(0, 0, 0, 0);
            }
        }
    }
#pragma unroll
    for (int tt = 0; tt < TT; ++tt)
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            float v = acc[tt][c];
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            if (kr == 0) red[(warp * TT + tt) * 32 + cg * 8 + c] = v;
        }
    __syncthreads();
    for (int i = tid; i < TT * 32; i += blockDim.x) {
        const int tt = i / 32, c = i % 32;
        if (t0 + tt < T && n0 + c < N) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) v += red[(w * TT + tt) * 32 + c];
            y[((size_t)(t0 + tt) * Hh + h) * N + n0 + c] = __float2bfloat16(v);
            red[tt * 32 + c] = v;            // warp 0's slot (only this thread reads or writes column c of row tt)
        }
    }
    if (xp == nullptr) return;
    __syncthreads();
    // the same values (rounded to bf16 first, as a separate staging pass would see them) as f16 units of 8
    const int Kt = Hh * N;
    for (int i = tid; i < TT * 4; i += blockDim.x) {
        const int tt = i / 4, c8 = (i % 4) * 8, tok = t0 + tt;
        if (n0 + c8 >= N) continue;
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float a = 0.f, b = 0.f;
            if (tok < T) {
                a = __bfloat162float(__float2bfloat16(red[tt * 32 + c8 + 2 * q]));
                b = __bfloat162float(__float2bfloat16(red[tt * 32 + c8 + 2 * q + 1]));
            }
            const __half2 hh = __floats2half2_rn(a, b);
            w[q] = *reinterpret_cast<const uint32_t*>(&hh);
        }
        const int u = (h * N + n0 + c8) / 8, group = u / 16, within = u % 16, cc = within / 4, j = within % 4;
        xp[((size_t)tok * (Kt / 128) + group) * 16 + j * 4 + cc] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

template <int TT>
__device__ __forceinline__ void bmv_body(bf16* __restrict__ y, const void* __restrict__ x, const bf16* __restrict__ M, int T,
                                         int Hh, int K, int N, int xs_t, int xs_h, int n_slabs, long long slab_stride, int h,
                                         int n0, int t0) {
    bmv_core<TT>(y, nullptr, M, T, Hh, K, N, h, n0, t0, [&](float* xs) {
        for (int i = threadIdx.x; i < TT * K; i += blockDim.x) {
            const int tt = i / K, kk = i % K;
            xs[i] = (t0 + tt < T) ? load_act(x, n_slabs, slab_stride, (size_t)(t0 + tt) * xs_t + (size_t)h * xs_h + kk) : 0.f;
        }
    });
}

// Attention output at decode: the merge of the key-split partial results (softmax weights from the partial
// log-sum-exps) is the staging step of the value expansion, so (o_part, lse_part) -> y = merge(o_part) x w_v[h] is one
// launch, and the rows leave in the operand order of the output projection as well.
// o_part [T, Hh, np, K] fp32, lse_part [T, Hh, np]; np <= 64; K % 4 == 0.
struct CombineExpandParams {
    const float* o_part; const float* lse_part;
    const bf16* w_v;          // [Hh, K, N]
    bf16* y;                  // [T, Hh * N]
    uint4* xp;                // fragment-ordered f16 copy [tpad, Hh * N], or null
    int T, tpad, Hh, K, N, np;
};

template <int TT>
__global__ void __launch_bounds__(256) combine_vexpand_kernel(CombineExpandParams p) {
    pdl_grid_sync();
    __shared__ float wsh[TT][64];
    __shared__ float s_inv[TT];
    const int h = blockIdx.x, n0 = blockIdx.y * 32, t0 = blockIdx.z * TT;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (warp < TT) {
        const int t = t0 + warp;
        float l0 = -INFINITY, l1 = -INFINITY;
        if (t < p.T) {
            const float* lp = p.lse_part + ((size_t)t * p.Hh + h) * p.np;
            if (lane < p.np) l0 = lp[lane];
            if (lane + 32 < p.np) l1 = lp[lane + 32];
        }
        const float mx = warp_max(fmaxf(l0, l1));
        const float w0 = l0 == -INFINITY ? 0.f : __expf(l0 - mx), w1 = l1 == -INFINITY ? 0.f : __expf(l1 - mx);
        const float den = warp_sum(w0) + warp_sum(w1);      // the order of the stand-alone merge kernel's sum
        wsh[warp][lane] = w0;
        wsh[warp][lane + 32] = w1;
        if (lane == 0) s_inv[warp] = den > 0.f ? 1.f / den : 0.f;
    }
    __syncthreads();
    bmv_core<TT>(p.y, p.xp, p.w_v, p.T, p.Hh, p.K, p.N, h, n0, t0, [&](float* xs) {
        const int k4 = p.K / 4;
        for (int i = tid; i < TT * k4; i += 256) {
            const int tt = i / k4, d = (i % k4) * 4, t = t0 + tt;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < p.T) {
                const float* op = p.o_part + ((size_t)t * p.Hh + h) * p.np * p.K + d;
                for (int i0 = 0; i0 < p.np; i0 += 8) {
                    float4 v[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) v[u] = *reinterpret_cast<const float4*>(op + (size_t)min(i0 + u, p.np - 1) * p.K);
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const float w = i0 + u < p.np ? wsh[tt][i0 + u] : 0.f;
                        acc.x += w * v[u].x; acc.y += w * v[u].y; acc.z += w * v[u].z; acc.w += w * v[u].w;
                    }
                }
                // the merged row is rounded to bf16, as the stand-alone merge kernel stores it
                const float inv = s_inv[tt];
                acc.x = __bfloat162float(__float2bfloat16(acc.x * inv)); acc.y = __bfloat162float(__float2bfloat16(acc.y * inv));
                acc.z = __bfloat162float(__float2bfloat16(acc.z * inv)); acc.w = __bfloat162float(__float2bfloat16(acc.w * inv));
            }
            *reinterpret_cast<float4*>(xs + tt * p.K + d) = acc;
        }
    });
}

template <int TT>
static int launch_combine_vexpand(const CombineExpandParams* p, cudaStream_t s) {
    const int rows = p->xp != nullptr ? p->tpad : p->T;
    dim3 grid(p->Hh, (p->N + 31) / 32, (rows + TT - 1) / TT);
    const size_t smem = (size_t)(TT * p->K + 8 * TT * 32) * sizeof(float);
    auto kern = combine_vexpand_kernel<TT>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sl_launch(kern, grid, 256, smem, s, *p);
    return SL_LAUNCH_CHECK();
}

SL_API int sl_combine_vexpand(const CombineExpandParams* p, cudaStream_t s) {
    if (p->T == 0) return 0;
    if (p->N % 8 != 0 || p->K % 4 != 0 || p->np < 1 || p->np > 64) return -1;
    if (p->xp != nullptr && ((p->Hh * p->N) % 128 != 0 || p->tpad % 8 != 0 || p->tpad < p->T)) return -1;
    if (p->T == 1) return launch_combine_vexpand<1>(p, s);
    if (p->T == 2) return launch_combine_vexpand<2>(p, s);
    return launch_combine_vexpand<4>(p, s);
}

template <int TT>
__global__ void __launch_bounds__(256) bmv_kernel(bf16* __restrict__ y, const void* __restrict__ x, const bf16* __restrict__ M,
                                                  int T, int Hh, int K, int N, int xs_t, int xs_h, int n_slabs,
                                                  long long slab_stride) {
    pdl_grid_sync();
    bmv_body<TT>(y, x, M, T, Hh, K, N, xs_t, xs_h, n_slabs, slab_stride, blockIdx.x, blockIdx.y * 32, blockIdx.z * TT);
}

// q_post and the absorb product (q_nope x W_kn) read the same projection and do not depend on each other: one
// launch, the first `bmv_blocks` blocks do the product, the rest the per-head rotary / quantisation work.
template <int TT>
__global__ void __launch_bounds__(256) q_post_absorb_kernel(QPostParams p, bf16* __restrict__ q_abs, const bf16* __restrict__ w_kn,
                                                            int T, int K, int N, int bmv_blocks, int col_chunks) {
    pdl_grid_sync();
    const int b = blockIdx.x;
    if (b < bmv_blocks) {
        const int h = b % p.heads, rest = b / p.heads, nc = rest % col_chunks, tz = rest / col_chunks;
        bmv_body<TT>(q_abs, p.qb, w_kn, T, p.heads, K, N, p.ld, p.d_nope + p.rope_dim, p.n_slabs, p.slab_stride, h, nc * 32, tz * TT);
    } else {
        const int i = b - bmv_blocks, per_t = p.heads + p.idx_heads;
        q_post_body(p, i / per_t, i % per_t);
    }
}

template <int TT>
static int launch_q_post_absorb(const QPostParams* p, void* q_abs, const void* w_kn, int T, int K, int N, cudaStream_t s) {
    const int col_chunks = (N + 31) / 32, tz = (T + TT - 1) / TT;
    const int bmv_blocks = p->heads * col_chunks * tz, post_blocks = T * (p->heads + p->idx_heads);
    const size_t smem = (size_t)(TT * K + 8 * TT * 32) * sizeof(float);
    auto kern = q_post_absorb_kernel<TT>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sl_launch(kern, bmv_blocks + post_blocks, 256, smem, s, *p, (bf16*)q_abs, (const bf16*)w_kn, T, K, N, bmv_blocks, col_chunks);
    return SL_LAUNCH_CHECK();
}

// q_post plus q_abs[t, h, :] = q_nope[t, h, :] x w_kn[h] (K = d_nope, N = kv_lora) in one launch.
SL_API int sl_q_post_absorb(const QPostParams* p, void* q_abs, const void* w_kn, int T, int N, cudaStream_t s) {
    if (T == 0) return 0;
    if (N % 8 != 0 || p->idx_dim > 512 || p->rope_dim > 512) return -1;
    const int K = p->d_nope;
    if (T == 1) return launch_q_post_absorb<1>(p, q_abs, w_kn, T, K, N, s);
    if (T == 2) return launch_q_post_absorb<2>(p, q_abs, w_kn, T, K, N, s);
    return launch_q_post_absorb<4>(p, q_abs, w_kn, T, K, N, s);
}

template <int TT>
static int launch_bmv(void* y, const void* x, const void* M, int T, int Hh, int K, int N, int xs_t, int xs_h, int n_slabs,
                      long long slab_stride, cudaStream_t s) {
    dim3 grid(Hh, (N + 31) / 32, (T + TT - 1) / TT);
    const size_t smem = (size_t)(TT * K + 8 * TT * 32) * sizeof(float);
    auto kern = bmv_kernel<TT>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sl_launch(kern, grid, 256, smem, s, (bf16*)y, x, (const bf16*)M, T, Hh, K, N, xs_t, xs_h, n_slabs, slab_stride);
    return SL_LAUNCH_CHECK();
}

// x is bf16, or (n_slabs > 0) a sum of fp32 slabs with the same element indexing (see load_act).
SL_API int sl_bmv(void* y, const void* x, const void* M, int T, int Hh, int K, int N, int xs_t, int xs_h, int n_slabs,
                  long long slab_stride, cudaStream_t s) {
    if (T == 0) return 0;
    if (N % 8 != 0) return -1;
    if (T == 1) return launch_bmv<1>(y, x, M, T, Hh, K, N, xs_t, xs_h, n_slabs, slab_stride, s);
    if (T == 2) return launch_bmv<2>(y, x, M, T, Hh, K, N, xs_t, xs_h, n_slabs, slab_stride, s);
    return launch_bmv<4>(y, x, M, T, Hh, K, N, xs_t, xs_h, n_slabs, slab_stride, s);
}

// ---------------------------------------------------------------------------------------------
// act[t, i] = silu(gu[t, i]) * gu[t, I + i]
__global__ void silu_mul_kernel(bf16* __restrict__ out, const bf16* __restrict__ gu, size_t total, int I) {
    pdl_grid_sync();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I, i = idx % I;
        const float g = __bfloat162float(gu[t * 2 * I + i]), u = __bfloat162float(gu[t * 2 * I + I + i]);
        out[idx] = __float2bfloat16(g / (1.f + __expf(-g)) * u);
    }
}

SL_API int sl_silu_mul(void* out, const void* gu, int T, int I, cudaStream_t s) {
    const size_t total = (size_t)T * I;
    if (total == 0) return 0;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    sl_launch(silu_mul_kernel, blocks, 256, 0, s, (bf16*)out, (const bf16*)gu, total, I);
    return SL_LAUNCH_CHECK();
}

// SwiGLU on f16 rows (the NVFP4 prefill GEMMs run in f16): out[t, i] = silu(gu[t, i]) * gu[t, I + i].
__global__ void silu_mul_h_kernel(__half* __restrict__ out, const __half* __restrict__ gu, size_t total_pairs, int I) {
    pdl_grid_sync();
    const int I2 = I / 2;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_pairs; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I2, i = (idx % I2) * 2;
        const float2 g = __half22float2(*reinterpret_cast<const __half2*>(gu + t * 2 * I + i));
        const float2 u = __half22float2(*reinterpret_cast<const __half2*>(gu + t * 2 * I + I + i));
        *reinterpret_cast<__half2*>(out + t * I + i) = __floats2half2_rn(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
    }
}

SL_API int sl_silu_mul_h(void* out, const void* gu, int T, int I, cudaStream_t s) {
    if (I % 2 != 0) return -1;
    const size_t total = (size_t)T * (I / 2);
    if (total == 0) return 0;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    sl_launch(silu_mul_h_kernel, blocks, 256, 0, s, (__half*)out, (const __half*)gu, total, I);
    return SL_LAUNCH_CHECK();
}

// out[m, :] = f16(x[src[m], :]) for bf16 x (src null: identity).  One warp per 256 columns of a row, 16-byte accesses.
__global__ void gather_rows_f16_kernel(__half* __restrict__ out, const bf16* __restrict__ x, const int* __restrict__ src, int M, int H,
                                       int ldx, int rows_x) {
    pdl_grid_sync();
    const int per_row = H / 8;                              // 16-byte pieces per row
    const size_t total = (size_t)M * per_row;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int m = (int)(idx / per_row), c = (int)(idx % per_row) * 8;
        const int r = src ? src[m] : m;
        uint4 o = make_uint4(0u, 0u, 0u, 0u);
        if (r >= 0 && r < rows_x) {
            const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)r * ldx + c);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t h[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = bf162_to_f2(w[i]);
                __half2 hv = __floats2half2_rn(f.x, f.y);
                h[i] = *reinterpret_cast<uint32_t*>(&hv);
            }
            o = make_uint4(h[0], h[1], h[2], h[3]);
        }
        *reinterpret_cast<uint4*>(out + (size_t)m * H + c) = o;
    }
}

SL_API int sl_gather_rows_f16(void* out, const void* x, const void* src, int M, int H, int ldx, int rows_x, cudaStream_t s) {
    if (M <= 0) return 0;
    if (H % 8 != 0 || ldx % 8 != 0) return -1;
    const size_t total = (size_t)M * (H / 8);
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    sl_launch(gather_rows_f16_kernel, blocks, 256, 0, s, (__half*)out, (const bf16*)x, (const int*)src, M, H, ldx, rows_x);
    return SL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// MoE routing: one warp per token (see route.cuh).
template <int PER>
__global__ void route_topk_kernel(int* __restrict__ ids, float* __restrict__ wts, const float* __restrict__ logits,
                                  const float* __restrict__ bias, int T, int E, int top_k, int n_group, int topk_group,
                                  int norm, float scale) {
    pdl_grid_sync();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= T) return;
    float lg[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = lane * PER + i;
        lg[i] = e < E ? logits[(size_t)warp * E + e] : 0.f;
    }
    int id; float w;
    route_warp<PER>(lg, bias, E, top_k, n_group, topk_group, norm, scale, id, w);
    if (lane < top_k) {
        ids[(size_t)warp * top_k + lane] = id;
        wts[(size_t)warp * top_k + lane] = w;
    }
}

SL_API int sl_route_topk(void* ids, void* wts, const void* logits, const void* bias, int T, int E, int top_k, int n_group,
                         int topk_group, int norm, float scale, cudaStream_t s) {
    if (T == 0) return 0;
    if (E > 512 || top_k > 32 || n_group > 32 || n_group < 1 || E % n_group != 0) return -1;
    const int per = (E + 31) / 32;
    int PER = 1;
    while (PER < per) PER <<= 1;
    if (n_group > 1) {
        const int gsz = E / n_group;
        if (gsz % PER != 0) return -1;                       // a group must be a run of whole lanes
        const int lpg = gsz / PER;
        if (lpg & (lpg - 1)) return -1;
    }
    const int wpb = 4;
    dim3 grid((T + wpb - 1) / wpb), block(wpb * 32);
#define SL_ROUTE(P) sl_launch(route_topk_kernel<P>, grid, block, 0, s, (int*)ids, (float*)wts, (const float*)logits, (const float*)bias, \
                                                                T, E, top_k, n_group, topk_group, norm, scale)
    switch (PER) {
        case 1: SL_ROUTE(1); break;
        case 2: SL_ROUTE(2); break;
        case 4: SL_ROUTE(4); break;
        case 8: SL_ROUTE(8); break;
        default: SL_ROUTE(16); break;
    }
#undef SL_ROUTE
    return SL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Global key positions -> this rank's physical slots, with ordered compaction of dropped
// entries (-1, or owned by another CP rank when local_only).  One block per token, k <= 4096.
__global__ void topk_to_slots_kernel(int* __restrict__ slots, int* __restrict__ lengths, const int* __restrict__ pos,
                                     const int* __restrict__ page_table, const int* __restrict__ batch_idx, int k,
                                     int pt_stride, int page_size, int cp_world, int cp_rank, int local_only, int* guard) {
    pdl_grid_sync();
    __shared__ int wsum[32];
    __shared__ int base;
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    const int* pt = page_table + (size_t)batch_idx[t] * pt_stride;
    if (tid == 0) base = 0;
    __syncthreads();
    for (int c0 = 0; c0 < k; c0 += blockDim.x) {
        const int i = c0 + tid;
        int p = (i < k) ? pos[(size_t)t * k + i] : -1;
        bool valid = p >= 0;
        if (valid && local_only && cp_world > 1 && (p % cp_world) != cp_rank) valid = false;
        const unsigned m = __ballot_sync(0xffffffffu, valid);
        const int inw = __popc(m & ((1u << lane) - 1));
        if (lane == 0) wsum[warp] = __popc(m);
        __syncthreads();
        int off = base;
        for (int w = 0; w < warp; ++w) off += wsum[w];
        if (valid) {
            const int local = p / cp_world;
            slots[(size_t)t * k + off + inw] =
                guard_ok(guard, 31, local / page_size, pt_stride) ? pt[local / page_size] * page_size + local % page_size : 0;
        }
        __syncthreads();
        if (tid == 0) {
            int tot = 0;
            for (int w = 0; w < nw; ++w) tot += wsum[w];
            base += tot;
        }
        __syncthreads();
    }
    for (int i = base + tid; i < k; i += blockDim.x) slots[(size_t)t * k + i] = -1;
    if (tid == 0) lengths[t] = base;
}

SL_API int sl_topk_to_slots(void* slots, void* lengths, const void* pos, const void* page_table, const void* batch_idx, int T,
                            int k, int pt_stride, int page_size, int cp_world, int cp_rank, int local_only, void* guard,
                            cudaStream_t s) {
    if (T == 0) return 0;
    sl_launch(topk_to_slots_kernel, T, 256, 0, s, (int*)slots, (int*)lengths, (const int*)pos, (const int*)page_table,
                                           (const int*)batch_idx, k, pt_stride, page_size, cp_world, cp_rank, local_only, (int*)guard);
    return SL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// MTP input shift: within each sequence ids[t] <- ids[t+1]; the last slot takes the new token.
// (reference `csrc/glm_ops.cu:3308`)
__global__ void rotate_input_ids_kernel(int64_t* __restrict__ out, const int64_t* __restrict__ ids,
                                        const int64_t* __restrict__ new_tokens, const int* __restrict__ qo_indptr, int B) {
    pdl_grid_sync();
    const int b = blockIdx.x;
    if (b >= B) return;
    const int lo = qo_indptr[b], hi = qo_indptr[b + 1];
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) out[i] = (i + 1 < hi) ? ids[i + 1] : new_tokens[b];
}

SL_API int sl_rotate_input_ids(void* out, const void* ids, const void* new_tokens, const void* qo_indptr, int B, cudaStream_t s) {
    if (B == 0) return 0;
    sl_launch(rotate_input_ids_kernel, B, 128, 0, s, (int64_t*)out, (const int64_t*)ids, (const int64_t*)new_tokens, (const int*)qo_indptr, B);
    return SL_LAUNCH_CHECK();
}
