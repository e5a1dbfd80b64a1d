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
template <int PER>
__device__ __forceinline__ void route_warp(const float (&logit)[PER], const float* __restrict__ bias, int E, int top_k,
                                           int n_group, int topk_group, int norm, float scale, int& out_id, float& out_w) {
    const int lane = threadIdx.x & 31;
    float sc[PER], ch[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = lane * PER + i;
        if (e < E) {
            const float s = 1.f / (1.f + expf(-logit[i]));
            sc[i] = s;
            ch[i] = s + (bias ? bias[e] : 0.f);
        } else {
            sc[i] = 0.f;
            ch[i] = -INFINITY;
        }
    }
    if (n_group > 1) {
        const int gsz = E / n_group;
        // top-2 of this lane's experts, merged across the lanes of its group
        float m1 = -INFINITY, m2 = -INFINITY;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const float v = ch[i];
            if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) m2 = v;
        }
        const int lanes_per_group = gsz / PER;            // >= 1 (checked by the launcher)
        for (int o = 1; o < lanes_per_group; o <<= 1) {
            const float o1 = __shfl_xor_sync(0xffffffffu, m1, o), o2 = __shfl_xor_sync(0xffffffffu, m2, o);
            const float hi = fmaxf(m1, o1), lo = fmaxf(fminf(m1, o1), fmaxf(m2, o2));
            m1 = hi; m2 = lo;
        }
        const int my_group = (lane * PER) / gsz;
        const float gs = gsz >= 2 ? m1 + m2 : m1;
        // rank of my group: number of groups that beat it (higher score, or equal score and lower id)
        int beaten_by = 0;
        for (int g2 = 0; g2 < n_group; ++g2) {
            const float og = __shfl_sync(0xffffffffu, gs, g2 * lanes_per_group);
            beaten_by += (og > gs) || (og == gs && g2 < my_group);
        }
        if (beaten_by >= topk_group || lane * PER >= E) {
#pragma unroll
            for (int i = 0; i < PER; ++i) ch[i] = -INFINITY;
        }
    }
    float wsum = 0.f, myw = 0.f;
    int myid = 0;
    for (int r = 0; r < top_k; ++r) {
        float best = -INFINITY; int bslot = 0;
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (ch[i] > best) { best = ch[i]; bslot = i; }
        const int be = best > -INFINITY ? lane * PER + bslot : E;
        float gb = best; int ge = be;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, gb, o);
            const int oe = __shfl_xor_sync(0xffffffffu, ge, o);
            if (ob > gb || (ob == gb && oe < ge)) { gb = ob; ge = oe; }
        }
        float s = 0.f;
        if (ge == be && be < E) {
#pragma unroll
            for (int i = 0; i < PER; ++i)
                if (i == bslot) { s = sc[i]; ch[i] = -INFINITY; }
        }
        // hand the winner's unbiased score to every lane
        s = __shfl_sync(0xffffffffu, s, ge < E ? ge / PER : 0);
        wsum += s;
        if (lane == r) { myw = s; myid = ge < E ? ge : 0; }
    }
    float w = myw;
    if (norm) w = w / fmaxf(wsum, 1e-20f);
    out_id = myid;
    out_w = w * scale;
}
