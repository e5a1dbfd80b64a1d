// Token sampling on the device: penalties, temperature, top-k (<= 64), top-p, counter RNG,
// candidate sets for speculative decoding and linear-chain rejection sampling.
//
// Reference: `csrc/glm_sampling.cu:276-400` (batched sampler), `:403` (argmax), `:557`
// (candidate sampling), `:644-706` (spec_reject_linear), `:54-70` (lowbias32 counter RNG).
#include "common.cuh"

#define SL_MAX_CAND 256

__device__ __forceinline__ uint32_t lowbias32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du;
    x ^= x >> 15; x *= 0x846ca68bu;
    x ^= x >> 16;
    return x;
}
// Uniform in (0,1) from (counter, row, stream); the Python reference computes the same value.
__device__ __forceinline__ double uniform_from_counter(uint32_t counter, uint32_t row, uint32_t stream) {
    const uint32_t h = lowbias32(lowbias32(row * 0x9E3779B1u + counter) + stream * 0x85EBCA6Bu);
    return ((double)h + 0.5) / 4294967296.0;
}
__device__ __forceinline__ uint32_t order_key_f(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// ---------------------------------------------------------------------------------------------
// Arg-max over the vocabulary in two stages: grid (chunks, B) partial winners, then one warp per
// row.  Ties go to the lower index; a row of NaN / -inf still yields a valid id (0).
#define SL_ARGMAX_CHUNKS 64
template <typename TL>
__global__ void __launch_bounds__(256) argmax_partial_kernel(float* __restrict__ pv, int* __restrict__ pi,
                                                             const TL* __restrict__ logits, int V, int ld) {
    pdl_grid_sync();
    __shared__ float sv[8];
    __shared__ int si[8];
    const int b = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per = (V + gridDim.x - 1) / gridDim.x;
    const int lo = blockIdx.x * per, hi = min(V, lo + per);
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = (float)logits[(size_t)b * ld + i];
        if (v > best) { best = v; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
        pv[(size_t)b * gridDim.x + blockIdx.x] = best;
        pi[(size_t)b * gridDim.x + blockIdx.x] = bi;
    }
}

__global__ void argmax_final_kernel(int64_t* __restrict__ out, float* __restrict__ out_val, const float* __restrict__ pv,
                                    const int* __restrict__ pi, int chunks, int64_t id_offset) {
    pdl_grid_sync();
    const int b = blockIdx.x, lane = threadIdx.x;
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int i = lane; i < chunks; i += 32) {
        const float v = pv[(size_t)b * chunks + i]; const int id = pi[(size_t)b * chunks + i];
        if (v > best || (v == best && id < bi)) { best = v; bi = id; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) {
        if (bi == 0x7fffffff) bi = 0;
        out[b] = (int64_t)bi + id_offset;
        if (out_val) out_val[b] = best;
    }
}

// scratch_val / scratch_idx: [B, 64] floats / ints owned by the caller.
SL_API int sl_argmax(void* out, const void* logits, int B, int V, int ld, int is_f32, long long id_offset, void* out_val,
                     void* scratch_val, void* scratch_idx, cudaStream_t s) {
    if (B == 0) return 0;
    dim3 grid(SL_ARGMAX_CHUNKS, B);
    if (is_f32) sl_launch(argmax_partial_kernel<float>, grid, 256, 0, s, (float*)scratch_val, (int*)scratch_idx, (const float*)logits, V, ld);
    else sl_launch(argmax_partial_kernel<bf16>, grid, 256, 0, s, (float*)scratch_val, (int*)scratch_idx, (const bf16*)logits, V, ld);
    sl_launch(argmax_final_kernel, B, 32, 0, s, (int64_t*)out, (float*)out_val, (const float*)scratch_val, (const int*)scratch_idx,
                                         SL_ARGMAX_CHUNKS, id_offset);
    return SL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
struct SampleParams {
    float* logits; int V, ld;            // [B, ld] fp32, modified in place by the penalties
    const float *temperature, *top_p, *rep_penalty, *presence_penalty;   // [B]
    const int* top_k;                    // [B] (<= 0: max_k)
    const int64_t* history; const int* hist_len; int window;             // [B, window]
    int max_k;                           // candidate capacity (<= 256)
    const uint32_t* counter;             // device word: RNG counter (advanced by sl_advance_counter)
    uint32_t stream;
    const int* row_ids;                  // RNG row id per batch row (null = row index)
    int64_t* out_token;                  // [B]
    int64_t* cand_ids; float* cand_probs;                                 // [B, max_k] or null
};

__global__ void __launch_bounds__(1024) sample_kernel(SampleParams p) {
    pdl_grid_sync();
    __shared__ uint32_t hist[256];
    __shared__ uint32_t s_prefix, s_remaining;
    __shared__ float cv[SL_MAX_CAND];
    __shared__ int ci[SL_MAX_CAND];
    __shared__ float sv[SL_MAX_CAND];
    __shared__ int sidx[SL_MAX_CAND];
    __shared__ int s_count;
    const int b = blockIdx.x, tid = threadIdx.x;
    float* lg = p.logits + (size_t)b * p.ld;

    // penalties over the recent-token window (each distinct token once)
    if (p.history != nullptr) {
        const int n = min(p.hist_len[b], p.window);
        const float rp = p.rep_penalty ? p.rep_penalty[b] : 1.f, pp = p.presence_penalty ? p.presence_penalty[b] : 0.f;
        if (tid < n && (rp != 1.f || pp != 0.f)) {
            const int64_t tok = p.history[(size_t)b * p.window + tid];
            bool first = tok >= 0 && tok < p.V;
            for (int i = 0; i < tid && first; ++i) first = p.history[(size_t)b * p.window + i] != tok;
            if (first) {
                float v = lg[tok];
                v = v > 0.f ? v / rp : v * rp;
                lg[tok] = v - pp;
            }
        }
        __syncthreads();
    }
    const float temp = p.temperature[b];
    int K = p.top_k[b] <= 0 ? p.max_k : min(p.top_k[b], p.max_k);
    if (temp <= 0.f) K = 1;
    K = min(K, p.V);

    // radix descent for the K-th largest logit
    uint32_t mask = 0;
    if (tid == 0) { s_prefix = 0; s_remaining = (uint32_t)K; s_count = 0; }
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = tid; i < 256; i += blockDim.x) hist[i] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        for (int i = tid; i < p.V; i += blockDim.x) {
            const uint32_t key = order_key_f(lg[i]);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            uint32_t rem = s_remaining, cum = 0;
            int bb = 255;
            for (; bb > 0; --bb) {
                if (cum + hist[bb] >= rem) break;
                cum += hist[bb];
            }
            s_remaining = rem - cum;
            s_prefix = prefix | ((uint32_t)bb << shift);
        }
        __syncthreads();
        mask |= 0xffu << shift;
    }
    const uint32_t thr = s_prefix;
    // gather: strictly greater first (any order), ties resolved afterwards by index
    for (int i = tid; i < p.V; i += blockDim.x) {
        const float v = lg[i];
        if (order_key_f(v) > thr) {
            const int slot = atomicAdd(&s_count, 1);
            if (slot < SL_MAX_CAND) { cv[slot] = v; ci[slot] = i; }
        }
    }
    __syncthreads();
    const int n_gt = min(s_count, K);
    __syncthreads();
    if (n_gt < K) {
        // ties with the threshold: take the lowest indices.  Sequential scan by warp 0 in index order.
        if (tid < 32) {
            int filled = n_gt;
            for (int base = 0; base < p.V && filled < K; base += 32) {
                const int i = base + tid;
                const bool eq = i < p.V && order_key_f(lg[i]) == thr;
                const unsigned m = __ballot_sync(0xffffffffu, eq);
                const int off = filled + __popc(m & ((1u << tid) - 1));
                if (eq && off < K) { cv[off] = lg[i]; ci[off] = i; }
                filled += __popc(m);
            }
        }
        __syncthreads();
    }
    // rank sort: descending value, ascending index
    if (tid < K) {
        const float v = cv[tid]; const int id = ci[tid];
        int rank = 0;
        for (int j = 0; j < K; ++j) rank += (cv[j] > v) || (cv[j] == v && ci[j] < id);
        sv[rank] = v; sidx[rank] = id;
    }
    __syncthreads();
    if (tid == 0) {
        const float t = fmaxf(temp, 1e-6f);
        const float mx = sv[0];
        float probs[SL_MAX_CAND];
        float den = 0.f;
        for (int j = 0; j < K; ++j) { probs[j] = expf((sv[j] - mx) / t); den += probs[j]; }
        const float tp = p.top_p ? p.top_p[b] : 1.f;
        float csum = 0.f, kept = 0.f;
        int nk = 0;
        for (int j = 0; j < K; ++j) {
            const float pj = probs[j] / den;
            if (csum < tp || j == 0) { kept += pj; nk = j + 1; probs[j] = pj; } else probs[j] = 0.f;
            csum += pj;
        }
        for (int j = 0; j < nk; ++j) probs[j] /= kept;
        const uint32_t row = p.row_ids ? (uint32_t)p.row_ids[b] : (uint32_t)b;
        const double u = uniform_from_counter(*p.counter, row, p.stream);
        double c = 0.0; int pick = nk - 1;
        for (int j = 0; j < nk; ++j) { c += (double)probs[j]; if (u < c) { pick = j; break; } }
        p.out_token[b] = sidx[pick];
        if (p.cand_ids) {
            for (int j = 0; j < p.max_k; ++j) {
                p.cand_ids[(size_t)b * p.max_k + j] = j < K ? sidx[j] : 0;
                p.cand_probs[(size_t)b * p.max_k + j] = j < nk ? probs[j] : 0.f;
            }
        }
    }
}

SL_API int sl_sample(const SampleParams* p, int B, cudaStream_t s) {
    if (B == 0) return 0;
    if (p->max_k > SL_MAX_CAND || p->window > 1024) return -1;
    sl_launch(sample_kernel, B, 1024, 0, s, *p);
    return SL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Linear-chain speculative rejection sampling; one thread per row (D <= 8, C <= 256).  Candidate lists are sorted by
// probability, so everything behind the last non-zero entry is skipped: the sums are the same to the bit (adding zeros
// changes nothing) and the work follows the number of live candidates (top-k, top-p), not the capacity.
struct SpecRejectParams {
    const int64_t* draft_tokens;                                     // [B, D]
    const int64_t* draft_ids; const float* draft_probs;              // [B, D, C]
    const int64_t* target_ids; const float* target_probs;            // [B, D+1, C]
    int D, C;
    const uint32_t* counter;
    int64_t* out_tokens;                                             // [B, D+1] (-1 padded)
    int* num_accepted;                                               // [B]
};

__device__ int pick_from(const int64_t* ids, const float* w, int C, double u, int64_t* out) {
    double tot = 0.0;
    for (int c = 0; c < C; ++c) tot += (double)w[c];
    double acc = 0.0; int last = 0;
    for (int c = 0; c < C; ++c) {
        if (w[c] > 0.f) { last = c; acc += (double)w[c]; if (u * tot < acc) { *out = ids[c]; return c; } }
    }
    *out = ids[last];
    return last;
}

__global__ void spec_reject_kernel(SpecRejectParams p, int B) {
    pdl_grid_sync();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    const int D = p.D, C = p.C;
    int i = 0;
    for (int j = 0; j <= D; ++j) p.out_tokens[(size_t)b * (D + 1) + j] = -1;
    for (; i < D; ++i) {
        const int64_t x = p.draft_tokens[(size_t)b * D + i];
        const int64_t* tid_ = p.target_ids + ((size_t)b * (D + 1) + i) * C;
        const float* tp = p.target_probs + ((size_t)b * (D + 1) + i) * C;
        const int64_t* did = p.draft_ids + ((size_t)b * D + i) * C;
        const float* dp = p.draft_probs + ((size_t)b * D + i) * C;
        int Ct = C, Cd = C;                        // live prefixes of the two lists
        while (Ct > 1 && tp[Ct - 1] <= 0.f) --Ct;
        while (Cd > 1 && dp[Cd - 1] <= 0.f) --Cd;
        float pt = 0.f, pd = 0.f;
        for (int c = 0; c < Ct; ++c) if (tid_[c] == x) pt += tp[c];
        for (int c = 0; c < Cd; ++c) if (did[c] == x) pd += dp[c];
        const double ua = uniform_from_counter(*p.counter, (uint32_t)b, 2u * i + 1u);
        if (pd > 0.f && ua < (double)fminf(1.f, pt / pd)) {
            p.out_tokens[(size_t)b * (D + 1) + i] = x;
            continue;
        }
        float res[SL_MAX_CAND];
        float rs = 0.f;
        for (int c = 0; c < Ct; ++c) {
            float d = 0.f;
            for (int e = 0; e < Cd; ++e) if (did[e] == tid_[c]) d += dp[e];
            res[c] = fmaxf(tp[c] - d, 0.f);
            rs += res[c];
        }
        if (rs <= 0.f) for (int c = 0; c < Ct; ++c) res[c] = tp[c];
        int64_t tok;
        pick_from(tid_, res, Ct, uniform_from_counter(*p.counter, (uint32_t)b, 2u * i + 2u), &tok);
        p.out_tokens[(size_t)b * (D + 1) + i] = tok;
        break;
    }
    if (i == D) {
        int64_t tok;
        pick_from(p.target_ids + ((size_t)b * (D + 1) + D) * C, p.target_probs + ((size_t)b * (D + 1) + D) * C, C,
                  uniform_from_counter(*p.counter, (uint32_t)b, 2u * D + 2u), &tok);
        p.out_tokens[(size_t)b * (D + 1) + D] = tok;
    }
    p.num_accepted[b] = i;
}

SL_API int sl_spec_reject(const SpecRejectParams* p, int B, cudaStream_t s) {
    if (B == 0) return 0;
    if (p->C > SL_MAX_CAND) return -1;
    sl_launch(spec_reject_kernel, (B + 63) / 64, 64, 0, s, *p, B);
    return SL_LAUNCH_CHECK();
}

// RNG counter += inc (one thread; keeps graph replays from repeating random numbers).
__global__ void advance_counter_kernel(uint32_t* counter, uint32_t inc) {
    pdl_grid_sync(); *counter += inc; }
SL_API int sl_advance_counter(void* counter, unsigned inc, cudaStream_t s) {
    sl_launch(advance_counter_kernel, 1, 1, 0, s, (uint32_t*)counter, inc);
    return SL_LAUNCH_CHECK();
}
