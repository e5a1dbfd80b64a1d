// MoE routing for one token by one warp (shared by the stand-alone routing kernel and the fused
// router kernel of the decode MoE path).
#pragma once
#include "common.cuh"

// scores = sigmoid(logits); choose by scores + bias inside the `topk_group` best groups (group
// rank = sum of its two best biased scores); weights = unbiased scores of the chosen, normalised,
// scaled.  Ties prefer the lower expert id.  Lane l holds the logits of experts l*PER ..
// l*PER+PER-1 (contiguous, so a group of E/n_group experts is a run of whole lanes when
// E/n_group >= PER).  E <= 32*PER <= 512, n_group <= 32, top_k <= 32.  On return lane r < top_k
// holds the r-th choice in (id, weight).  Reference: `route_top8` (`csrc/glm_ops.cu:2343`).
template <int PER, int NT>
__device__ __forceinline__ void route_warp_n(const float (&logit)[NT][PER], const float* __restrict__ bias, int E, int top_k,
                                             int n_group, int topk_group, int norm, float scale, int (&out_id)[NT],
                                             float (&out_w)[NT]) {
    // NT tokens at once: their shuffle chains are independent, so the warp overlaps their latencies
    const int lane = threadIdx.x & 31;
    float sc[NT][PER], ch[NT][PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = lane * PER + i;
        const float b = (e < E && bias) ? bias[e] : 0.f;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            if (e < E) {
                const float s = 1.f / (1.f + expf(-logit[n][i]));
                sc[n][i] = s;
                ch[n][i] = s + b;
            } else {
                sc[n][i] = 0.f;
                ch[n][i] = -INFINITY;
            }
        }
    }
    if (n_group > 1) {
        const int gsz = E / n_group;
        // top-2 of this lane's experts, merged across the lanes of its group
        float m1[NT], m2[NT];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            m1[n] = m2[n] = -INFINITY;
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const float v = ch[n][i];
                if (v > m1[n]) { m2[n] = m1[n]; m1[n] = v; } else if (v > m2[n]) m2[n] = v;
            }
        }
        const int lanes_per_group = gsz / PER;            // >= 1 (checked by the launcher)
        for (int o = 1; o < lanes_per_group; o <<= 1) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const float o1 = __shfl_xor_sync(0xffffffffu, m1[n], o), o2 = __shfl_xor_sync(0xffffffffu, m2[n], o);
                const float hi = fmaxf(m1[n], o1), lo = fmaxf(fminf(m1[n], o1), fmaxf(m2[n], o2));
                m1[n] = hi; m2[n] = lo;
            }
        }
        const int my_group = (lane * PER) / gsz;
        float gs[NT];
        int beaten_by[NT];
#pragma unroll
        for (int n = 0; n < NT; ++n) { gs[n] = gsz >= 2 ? m1[n] + m2[n] : m1[n]; beaten_by[n] = 0; }
        // rank of my group: number of groups that beat it (higher score, or equal score and lower id)
        for (int g2 = 0; g2 < n_group; ++g2) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const float og = __shfl_sync(0xffffffffu, gs[n], g2 * lanes_per_group);
                beaten_by[n] += (og > gs[n]) || (og == gs[n] && g2 < my_group);
            }
        }
#pragma unroll
        for (int n = 0; n < NT; ++n)
            if (beaten_by[n] >= topk_group || lane * PER >= E) {
#pragma unroll
                for (int i = 0; i < PER; ++i) ch[n][i] = -INFINITY;
            }
    }
    float wsum[NT], myw[NT];
    unsigned taken[NT];                      // bit i: this lane's i-th expert has been chosen
#pragma unroll
    for (int n = 0; n < NT; ++n) { wsum[n] = 0.f; myw[n] = 0.f; out_id[n] = 0; taken[n] = 0u; }
    for (int r = 0; r < top_k; ++r) {
        float gb[NT], s[NT];
        int ge[NT], be[NT], bslot[NT];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            float best = -INFINITY;
            bslot[n] = 0;
            s[n] = 0.f;
#pragma unroll
            for (int i = 0; i < PER; ++i)
                if (!((taken[n] >> i) & 1u) && ch[n][i] > best) { best = ch[n][i]; bslot[n] = i; s[n] = sc[n][i]; }
            be[n] = best > -INFINITY ? lane * PER + bslot[n] : E;
            gb[n] = best; ge[n] = be[n];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const float ob = __shfl_xor_sync(0xffffffffu, gb[n], o);
                const int oe = __shfl_xor_sync(0xffffffffu, ge[n], o);
                if (ob > gb[n] || (ob == gb[n] && oe < ge[n])) { gb[n] = ob; ge[n] = oe; }
            }
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            if (ge[n] == be[n] && be[n] < E) taken[n] |= 1u << bslot[n]; else s[n] = 0.f;
            // hand the winner's unbiased score to every lane
            s[n] = __shfl_sync(0xffffffffu, s[n], ge[n] < E ? ge[n] / PER : 0);
            wsum[n] += s[n];
            if (lane == r) { myw[n] = s[n]; out_id[n] = ge[n] < E ? ge[n] : 0; }
        }
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        float w = myw[n];
        if (norm) w = w / fmaxf(wsum[n], 1e-20f);
        out_w[n] = w * scale;
    }
}

template <int PER>
__device__ __forceinline__ void route_warp(const float (&logit)[PER], const float* __restrict__ bias, int E, int top_k,
                                           int n_group, int topk_group, int norm, float scale, int& out_id, float& out_w) {
    float lg[1][PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) lg[0][i] = logit[i];
    int id[1];
    float w[1];
    route_warp_n<PER, 1>(lg, bias, E, top_k, n_group, topk_group, norm, scale, id, w);
    out_id = id[0];
    out_w = w[0];
}
