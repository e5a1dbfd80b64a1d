// Recurrent sub-layers of the hybrid model families (sm_100a, CUDA cores: the work is a rank-1
// state update per token, bandwidth- and latency-bound, not GEMM-shaped).
//
//  * Gated DeltaNet (Qwen3.5 linear-attention layers): single-token step and sequence scan with
//    the [dk, dv] state column of each thread held in registers; depthwise causal conv1d with
//    rolling state; gated RMSNorm.  Reference: `csrc/glm_gdn.cu:68` (step), `:208` (prefill),
//    `:359/:440` (conv), `:495` (gated norm).
//  * KDA (per-channel decay) scan, sigmoid-gated norm and the manifold hyper-connection kernels
//    of glm5_next.  Reference: `csrc/glm_flash_hybrid.cu:31-198`.
//
// Layouts: projections are token-major [T, C]; the q|k|v channels of the conv output are
// [h*dk | h*dk | h*dv]; recurrent state is fp32 [slot, h, dk, dv]; conv state is [slot, C, Kw-1].
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float x) {
    if (x > 20.f) return x;
    if (x < -20.f) return __expf(x);
    return log1pf(__expf(x));
}
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x * sigmoid_f(x); }

struct GdnParams {
    bf16* out;                 // [T, h, dv]
    float* state;              // [slots, h, dk, dv]
    const bf16* qkv;           // [T, ld_qkv]
    int ld_qkv;
    const bf16* a;             // [T, h]   (GDN: decay input; KDA: unused)
    const bf16* b;             // [T, h]   beta input
    const float* A_log;        // [h]
    const float* dt_bias;      // [h]
    const bf16* g;             // KDA: per-channel forget input [T, h, dk] (null for GDN); dt_bias is then [h, dk]
    const int* qo_indptr;      // [B + 1] token ranges of the sequences
    const int* state_idx;      // [B] state slot of each sequence
    int h, dk, dv;
    int normalize_qk;          // L2-normalise q (then scale dk^-0.5) and k
    float lower_bound;         // KDA: decay = exp(lower_bound * sigmoid(exp(A_log[h]) * (forget + dt_bias)))
    float norm_eps;            // added to the squared norms (GDN 1e-8, KDA 1e-6)
};

// One block per (sequence, head); thread j owns state column S[:, j] (dv <= blockDim.x), kept in
// registers over the whole token range.  DK is the compile-time key dimension.
template <int DK>
__global__ void __launch_bounds__(128) delta_scan_kernel(GdnParams p) {
    pdl_grid_sync();
    __shared__ float s_q[DK], s_k[DK], s_g[DK];
    __shared__ float s_red[8];
    __shared__ float s_scal[2];
    const int seq = blockIdx.x / p.h, h = blockIdx.x % p.h, tid = threadIdx.x;
    const int t_begin = p.qo_indptr[seq], t_end = p.qo_indptr[seq + 1];
    if (t_begin >= t_end) return;
    const int j = tid;
    const bool active = j < p.dv;
    float* Sg = p.state + (((size_t)p.state_idx[seq] * p.h + h) * DK) * p.dv;
    float S[DK];
#pragma unroll
    for (int i = 0; i < DK; ++i) S[i] = active ? Sg[(size_t)i * p.dv + j] : 0.f;
    const int qoff = h * DK, koff = p.h * DK + h * DK, voff = 2 * p.h * DK + h * p.dv;
    for (int t = t_begin; t < t_end; ++t) {
        const bf16* row = p.qkv + (size_t)t * p.ld_qkv;
        __syncthreads();
        float qq = 0.f, kk = 0.f;
        for (int i = tid; i < DK; i += blockDim.x) {
            const float q = __bfloat162float(row[qoff + i]), k = __bfloat162float(row[koff + i]);
            s_q[i] = q; s_k[i] = k;
            qq += q * q; kk += k * k;
            if (p.g != nullptr)
                s_g[i] = __expf(p.lower_bound * sigmoid_f(__expf(p.A_log[h]) * (__bfloat162float(p.g[((size_t)t * p.h + h) * DK + i]) +
                                                                              p.dt_bias[h * DK + i])));
        }
        if (p.normalize_qk) {
            qq = warp_sum(qq); kk = warp_sum(kk);
            if ((tid & 31) == 0) { s_red[(tid >> 5) * 2] = qq; s_red[(tid >> 5) * 2 + 1] = kk; }
        }
        if (tid == 0) {
            // KDA: the beta logits are bf16 and so is their sigmoid in the checkpoint's definition
            const float bsig = sigmoid_f(__bfloat162float(p.b[(size_t)t * p.h + h]));
            s_scal[0] = p.g != nullptr ? __bfloat162float(__float2bfloat16(bsig)) : bsig;
            s_scal[1] = p.g != nullptr ? 1.f
                                       : __expf(-__expf(p.A_log[h]) * softplus_f(__bfloat162float(p.a[(size_t)t * p.h + h]) + p.dt_bias[h]));
        }
        __syncthreads();
        float qs = 1.f, ks = 1.f;
        if (p.normalize_qk) {
            float q2 = 0.f, k2 = 0.f;
            for (int w = 0; w < (int)(blockDim.x >> 5); ++w) { q2 += s_red[w * 2]; k2 += s_red[w * 2 + 1]; }
            qs = rsqrtf(q2 + p.norm_eps) * rsqrtf((float)DK);
            ks = rsqrtf(k2 + p.norm_eps);
        }
        const float beta = s_scal[0], decay = s_scal[1];
        if (active) {
            const float v = __bfloat162float(row[voff + j]);
            float kv = 0.f;
            if (p.g != nullptr) {
#pragma unroll
                for (int i = 0; i < DK; ++i) { S[i] *= s_g[i]; kv += S[i] * s_k[i]; }
            } else {
#pragma unroll
                for (int i = 0; i < DK; ++i) { S[i] *= decay; kv += S[i] * s_k[i]; }
            }
            const float delta = beta * (v - kv * ks);
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < DK; ++i) { S[i] += s_k[i] * ks * delta; o += S[i] * s_q[i]; }
            p.out[((size_t)t * p.h + h) * p.dv + j] = __float2bfloat16(o * qs);
        }
    }
    if (active) {
#pragma unroll
        for (int i = 0; i < DK; ++i) Sg[(size_t)i * p.dv + j] = S[i];
    }
}

// ---- causal depthwise conv1d over token-major activations -----------------------------------------
// y[t, c] = silu(sum_{w} W[c, w] * x[t - (Kw-1) + w, c] + bias[c]); inputs before the start of a
// sequence come from its rolling state [slot, C, Kw-1], which is then advanced.  One thread per
// (sequence, channel) walks the sequence's tokens (Kw <= 8).
__global__ void causal_conv1d_kernel(bf16* __restrict__ y, float* __restrict__ state, const bf16* __restrict__ x,
                                     const bf16* __restrict__ w, const bf16* __restrict__ bias, const int* __restrict__ qo_indptr,
                                     const int* __restrict__ state_idx, int B, int C, int Kw, int ldx, int activation) {
    pdl_grid_sync();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, seq = blockIdx.y;
    if (c >= C || seq >= B) return;
    const int t0 = qo_indptr[seq], t1 = qo_indptr[seq + 1];
    float* st = state + ((size_t)state_idx[seq] * C + c) * (Kw - 1);
    float win[8], wt[8];
    for (int i = 0; i < Kw - 1; ++i) win[i] = st[i];
    for (int i = 0; i < Kw; ++i) wt[i] = __bfloat162float(w[(size_t)c * Kw + i]);
    const float bv = bias != nullptr ? __bfloat162float(bias[c]) : 0.f;
    for (int t = t0; t < t1; ++t) {
        win[Kw - 1] = __bfloat162float(x[(size_t)t * ldx + c]);
        float acc = bv;
        for (int i = 0; i < Kw; ++i) acc += wt[i] * win[i];
        y[(size_t)t * C + c] = __float2bfloat16(activation ? silu_f(acc) : acc);
        for (int i = 0; i < Kw - 1; ++i) win[i] = win[i + 1];
    }
    for (int i = 0; i < Kw - 1; ++i) st[i] = win[i];
}

// out[r, :] = rmsnorm(x[r, :]) * w * act(gate[r, :]);  act = silu (GDN) or sigmoid (KDA).  One warp per row.
__global__ void rmsnorm_gated_kernel(bf16* __restrict__ out, const bf16* __restrict__ x, const bf16* __restrict__ gate,
                                     const bf16* __restrict__ w, int rows, int D, float eps, int sigmoid_gate) {
    pdl_grid_sync();
    const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (r >= rows) return;
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) {
        const float v = __bfloat162float(x[(size_t)r * D + i]);
        ss += v * v;
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)D + eps);
    for (int i = lane; i < D; i += 32) {
        const float v = __bfloat162float(x[(size_t)r * D + i]) * inv * __bfloat162float(w[i]);
        const float g = __bfloat162float(gate[(size_t)r * D + i]);
        out[(size_t)r * D + i] = __float2bfloat16(v * (sigmoid_gate ? sigmoid_f(g) : silu_f(g)));
    }
}

// ---- manifold hyper-connections: 4 residual streams per token -------------------------------------------
// pre: 24 coefficient logits = (x / rms(x)) . fn[c] over the 4*H values of the token (fp32), then
//   pre[i]  = sigmoid(l[i] * scale[0] + base[i]) + hc_eps                 (collapse weights)
//   post[i] = 2 * sigmoid(l[4+i] * scale[1] + base[4+i])                  (expansion weights)
//   comb    = Sinkhorn(softmax_rows(l[8..24] * scale[2] + base[8..24]) + hc_eps)
//   collapsed[d] = sum_s pre[s] * x[s, d]
// One block of 256 threads per token: each warp computes three of the 24 dot products.
__global__ void __launch_bounds__(256) mhc_pre_kernel(bf16* __restrict__ collapsed, float* __restrict__ post, float* __restrict__ comb,
                                                      const bf16* __restrict__ x, const bf16* __restrict__ fn,
                                                      const float* __restrict__ base, const float* __restrict__ scale, int H,
                                                      float norm_eps, float hc_eps, int iters) {
    pdl_grid_sync();
    __shared__ float scratch[33];
    __shared__ float logits[24], pre[4], mix[16];
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, width = 4 * H;
    const bf16* xr = x + (size_t)t * width;
    float ss = 0.f;
    for (int i = tid; i < width; i += blockDim.x) {
        const float v = __bfloat162float(xr[i]);
        ss += v * v;
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)width + norm_eps);
    for (int c = warp * 3; c < warp * 3 + 3; ++c) {
        float dot = 0.f;
        for (int i = lane; i < width; i += 32) dot += (__bfloat162float(xr[i]) * inv) * __bfloat162float(fn[(size_t)c * width + i]);
        dot = warp_sum(dot);
        if (lane == 0) logits[c] = dot;
    }
    __syncthreads();
    if (tid == 0) {
        for (int i = 0; i < 4; ++i) {
            pre[i] = sigmoid_f(logits[i] * scale[0] + base[i]) + hc_eps;
            post[t * 4 + i] = 2.f * sigmoid_f(logits[4 + i] * scale[1] + base[4 + i]);
        }
        for (int i = 0; i < 4; ++i) {
            float mx = -INFINITY, den = 0.f;
            for (int j = 0; j < 4; ++j) {
                mix[i * 4 + j] = logits[8 + i * 4 + j] * scale[2] + base[8 + i * 4 + j];
                mx = fmaxf(mx, mix[i * 4 + j]);
            }
            for (int j = 0; j < 4; ++j) { mix[i * 4 + j] = expf(mix[i * 4 + j] - mx); den += mix[i * 4 + j]; }
            for (int j = 0; j < 4; ++j) mix[i * 4 + j] = mix[i * 4 + j] / den + hc_eps;
        }
        for (int it = 0; it < iters; ++it) {
            if (it > 0) {
                for (int i = 0; i < 4; ++i) {
                    float den = hc_eps;
                    for (int j = 0; j < 4; ++j) den += mix[i * 4 + j];
                    for (int j = 0; j < 4; ++j) mix[i * 4 + j] /= den;
                }
            }
            for (int j = 0; j < 4; ++j) {
                float den = hc_eps;
                for (int i = 0; i < 4; ++i) den += mix[i * 4 + j];
                for (int i = 0; i < 4; ++i) mix[i * 4 + j] /= den;
            }
        }
        for (int i = 0; i < 16; ++i) comb[t * 16 + i] = mix[i];
    }
    __syncthreads();
    for (int d = tid; d < H; d += blockDim.x) {
        float v = 0.f;
        for (int sidx = 0; sidx < 4; ++sidx) v += pre[sidx] * __bfloat162float(xr[sidx * H + d]);
        collapsed[(size_t)t * H + d] = __float2bfloat16(v);
    }
}

// post: out[t, s, :] = post[t, s] * block[t, :] + sum_i comb[t, i, s] * residual[t, i, :]
__global__ void mhc_post_kernel(bf16* __restrict__ out, const bf16* __restrict__ residual, const bf16* __restrict__ block,
                                const float* __restrict__ post, const float* __restrict__ comb, int H) {
    pdl_grid_sync();
    const int t = blockIdx.x, sidx = blockIdx.y;
    float cw[4];
    for (int i = 0; i < 4; ++i) cw[i] = comb[t * 16 + i * 4 + sidx];
    const float pw = post[t * 4 + sidx];
    for (int d = threadIdx.x; d < H; d += blockDim.x) {
        float v = pw * __bfloat162float(block[(size_t)t * H + d]);
        for (int i = 0; i < 4; ++i) v += cw[i] * __bfloat162float(residual[((size_t)t * 4 + i) * H + d]);
        out[((size_t)t * 4 + sidx) * H + d] = __float2bfloat16(v);
    }
}

// expand: copy a [T, H] activation into 4 streams; collapse: mean of the 4 streams
__global__ void mhc_streams_kernel(bf16* __restrict__ out, const bf16* __restrict__ x, int H, int expand) {
    pdl_grid_sync();
    const int t = blockIdx.x;
    for (int d = threadIdx.x; d < H; d += blockDim.x) {
        if (expand) {
            const bf16 v = x[(size_t)t * H + d];
            for (int sidx = 0; sidx < 4; ++sidx) out[((size_t)t * 4 + sidx) * H + d] = v;
        } else {
            float v = 0.f;
            for (int sidx = 0; sidx < 4; ++sidx) v += __bfloat162float(x[((size_t)t * 4 + sidx) * H + d]);
            out[(size_t)t * H + d] = __float2bfloat16(v * 0.25f);
        }
    }
}

}  // namespace

// Gated DeltaNet / KDA scan over the token ranges qo_indptr[b] .. qo_indptr[b+1] of B sequences (a decode step is
// the case of one token per sequence).  dk in {64, 128}, dv <= 128.
SL_API int sl_delta_scan(const GdnParams* p, int B, cudaStream_t s) {
    if (B == 0) return 0;
    if (p->dv > 128) return -1;
    if (p->dk == 128) sl_launch(delta_scan_kernel<128>, B * p->h, 128, 0, s, *p);
    else if (p->dk == 64) sl_launch(delta_scan_kernel<64>, B * p->h, 128, 0, s, *p);
    else return -1;
    return SL_LAUNCH_CHECK();
}

SL_API int sl_causal_conv1d(void* y, void* state, const void* x, const void* w, const void* bias, const void* qo_indptr,
                            const void* state_idx, int B, int C, int Kw, int ldx, int activation, cudaStream_t s) {
    if (B == 0 || C == 0) return 0;
    if (Kw < 2 || Kw > 8) return -1;
    sl_launch(causal_conv1d_kernel, dim3((C + 127) / 128, B), 128, 0, s, (bf16*)y, (float*)state, (const bf16*)x, (const bf16*)w,
              (const bf16*)bias, (const int*)qo_indptr, (const int*)state_idx, B, C, Kw, ldx, activation);
    return SL_LAUNCH_CHECK();
}

SL_API int sl_rmsnorm_gated(void* out, const void* x, const void* gate, const void* w, int rows, int D, float eps,
                            int sigmoid_gate, cudaStream_t s) {
    if (rows == 0) return 0;
    sl_launch(rmsnorm_gated_kernel, (rows + 3) / 4, 128, 0, s, (bf16*)out, (const bf16*)x, (const bf16*)gate, (const bf16*)w, rows, D,
              eps, sigmoid_gate);
    return SL_LAUNCH_CHECK();
}

SL_API int sl_mhc_pre(void* collapsed, void* post, void* comb, const void* x, const void* fn, const void* base, const void* scale,
                      int T, int H, float norm_eps, float hc_eps, int iters, cudaStream_t s) {
    if (T == 0) return 0;
    if (iters < 1) return -1;
    sl_launch(mhc_pre_kernel, T, 256, 0, s, (bf16*)collapsed, (float*)post, (float*)comb, (const bf16*)x, (const bf16*)fn,
              (const float*)base, (const float*)scale, H, norm_eps, hc_eps, iters);
    return SL_LAUNCH_CHECK();
}

SL_API int sl_mhc_post(void* out, const void* residual, const void* block, const void* post, const void* comb, int T, int H,
                       cudaStream_t s) {
    if (T == 0) return 0;
    sl_launch(mhc_post_kernel, dim3(T, 4), 256, 0, s, (bf16*)out, (const bf16*)residual, (const bf16*)block, (const float*)post,
              (const float*)comb, H);
    return SL_LAUNCH_CHECK();
}

SL_API int sl_mhc_streams(void* out, const void* x, int T, int H, int expand, cudaStream_t s) {
    if (T == 0) return 0;
    sl_launch(mhc_streams_kernel, T, 256, 0, s, (bf16*)out, (const bf16*)x, H, expand);
    return SL_LAUNCH_CHECK();
}
