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
    const bf16* g;             // KDA: per-channel log decay [T, h, dk] (null for GDN)
    const int* qo_indptr;      // [B + 1] token ranges of the sequences
    const int* state_idx;      // [B] state slot of each sequence
    int h, dk, dv;
    int normalize_qk;          // GDN: L2-normalise q (then scale dk^-0.5) and k
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
            if (p.g != nullptr) s_g[i] = __expf(__bfloat162float(p.g[((size_t)t * p.h + h) * DK + i]));
        }
        if (p.normalize_qk) {
            qq = warp_sum(qq); kk = warp_sum(kk);
            if ((tid & 31) == 0) { s_red[(tid >> 5) * 2] = qq; s_red[(tid >> 5) * 2 + 1] = kk; }
        }
        if (tid == 0) {
            s_scal[0] = sigmoid_f(__bfloat162float(p.b[(size_t)t * p.h + h]));
            s_scal[1] = p.g != nullptr ? 1.f
                                       : __expf(-__expf(p.A_log[h]) * softplus_f(__bfloat162float(p.a[(size_t)t * p.h + h]) + p.dt_bias[h]));
        }
        __syncthreads();
        float qs = 1.f, ks = 1.f;
        if (p.normalize_qk) {
            float q2 = 0.f, k2 = 0.f;
            for (int w = 0; w < (int)(blockDim.x >> 5); ++w) { q2 += s_red[w * 2]; k2 += s_red[w * 2 + 1]; }
            qs = rsqrtf(q2 + 1e-8f) * rsqrtf((float)DK);
            ks = rsqrtf(k2 + 1e-8f);
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

// ---- manifold hyper-connections (n <= 8 residual streams) ----------------------------------------------
// pre: M = sinkhorn(exp(mix_logits[t])), mixed = M x streams[t], x = softmax(collapse_w[t]) . mixed.
// One block per token.
__global__ void mhc_pre_kernel(float* __restrict__ mixed, bf16* __restrict__ x, const float* __restrict__ streams,
                               const float* __restrict__ mix_logits, const float* __restrict__ collapse_w, int n, int H, int iters) {
    pdl_grid_sync();
    __shared__ float M[64], cw[8];
    const int t = blockIdx.x, tid = threadIdx.x;
    if (tid == 0) {
        float mx = -INFINITY;
        for (int i = 0; i < n * n; ++i) mx = fmaxf(mx, mix_logits[(size_t)t * n * n + i]);
        for (int i = 0; i < n * n; ++i) M[i] = __expf(mix_logits[(size_t)t * n * n + i] - mx);
        for (int it = 0; it < iters; ++it) {
            for (int r = 0; r < n; ++r) {
                float s = 0.f;
                for (int c = 0; c < n; ++c) s += M[r * n + c];
                for (int c = 0; c < n; ++c) M[r * n + c] /= s;
            }
            for (int c = 0; c < n; ++c) {
                float s = 0.f;
                for (int r = 0; r < n; ++r) s += M[r * n + c];
                for (int r = 0; r < n; ++r) M[r * n + c] /= s;
            }
        }
        float cm = -INFINITY, cs = 0.f;
        for (int i = 0; i < n; ++i) cm = fmaxf(cm, collapse_w[(size_t)t * n + i]);
        for (int i = 0; i < n; ++i) { cw[i] = __expf(collapse_w[(size_t)t * n + i] - cm); cs += cw[i]; }
        for (int i = 0; i < n; ++i) cw[i] /= cs;
    }
    __syncthreads();
    for (int d = tid; d < H; d += blockDim.x) {
        float s[8], xo = 0.f;
        for (int jn = 0; jn < n; ++jn) s[jn] = streams[((size_t)t * n + jn) * H + d];
        for (int i = 0; i < n; ++i) {
            float m = 0.f;
            for (int jn = 0; jn < n; ++jn) m += M[i * n + jn] * s[jn];
            mixed[((size_t)t * n + i) * H + d] = m;
            xo += cw[i] * m;
        }
        x[(size_t)t * H + d] = __float2bfloat16(xo);
    }
}

// post: streams_out[t, i, :] = mixed[t, i, :] + expand_w[t, i] * y[t, :]
__global__ void mhc_post_kernel(float* __restrict__ out, const float* __restrict__ mixed, const bf16* __restrict__ y,
                                const float* __restrict__ expand_w, int n, int H, size_t total) {
    pdl_grid_sync();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t d = idx % H, ti = idx / H, t = ti / n;
        out[idx] = mixed[idx] + expand_w[ti] * __bfloat162float(y[t * H + d]);
    }
}

// final collapse: mean over the streams
__global__ void mhc_streams_kernel(bf16* __restrict__ out, const float* __restrict__ streams, int n, int H, size_t total) {
    pdl_grid_sync();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t d = idx % H, t = idx / H;
        float s = 0.f;
        for (int i = 0; i < n; ++i) s += streams[(t * n + i) * H + d];
        out[idx] = __float2bfloat16(s / (float)n);
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

SL_API int sl_mhc_pre(void* mixed, void* x, const void* streams, const void* mix_logits, const void* collapse_w, int T, int n,
                      int H, int iters, cudaStream_t s) {
    if (T == 0) return 0;
    if (n > 8 || n < 1) return -1;
    sl_launch(mhc_pre_kernel, T, 256, 0, s, (float*)mixed, (bf16*)x, (const float*)streams, (const float*)mix_logits,
              (const float*)collapse_w, n, H, iters);
    return SL_LAUNCH_CHECK();
}

SL_API int sl_mhc_post(void* out, const void* mixed, const void* y, const void* expand_w, int T, int n, int H, cudaStream_t s) {
    if (T == 0) return 0;
    const size_t total = (size_t)T * n * H;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    sl_launch(mhc_post_kernel, blocks, 256, 0, s, (float*)out, (const float*)mixed, (const bf16*)y, (const float*)expand_w, n, H, total);
    return SL_LAUNCH_CHECK();
}

SL_API int sl_mhc_streams(void* out, const void* streams, int T, int n, int H, cudaStream_t s) {
    if (T == 0) return 0;
    const size_t total = (size_t)T * H;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    sl_launch(mhc_streams_kernel, blocks, 256, 0, s, (bf16*)out, (const float*)streams, n, H, total);
    return SL_LAUNCH_CHECK();
}
