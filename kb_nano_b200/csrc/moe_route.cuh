// Expert routing, warp-level: scores (softmax or sigmoid of the router logits), optional selection bias, optional
// group-limited selection, top-k, renormalisation and scaling for one token per warp.  Used by the stand-alone routing
// kernel and by the expert-parallel dispatch kernel when it routes on the way.
#pragma once
#include "common.cuh"

namespace kbn {

constexpr int kRouteMaxPerLane = 32;      // experts per lane: E <= 1024

__device__ __forceinline__ void argmax_merge(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) {
        v = ov;
        i = oi;
    }
}

// Routing arguments shared by the stand-alone kernel and the expert-parallel dispatch kernel that routes on the way.
struct RouteArgs {
    const void* logits;
    int64_t ld;
    int E, softmax;
    const float* bias;
    int n_group, topk_group, topk, renorm;
    float renorm_floor, scale;
    int round_bf16;
};

// One warp routes token t: on return lane r < topk holds the r-th choice (weight, expert id).
// PER = ceil(E / 32) rounded up to a power of two by the host (compile-time unrolling); expert of slot (j, lane)
// is j * 32 + lane.
template <int PER, bool BF16_IN>
__device__ __forceinline__ void route_token(const RouteArgs& a, int64_t t, int lane, float& out_weight, int& out_id) {
    const void* logits = a.logits;
    const int64_t ld = a.ld;
    const int E = a.E, softmax = a.softmax, n_group = a.n_group, topk_group = a.topk_group, topk = a.topk, renorm = a.renorm;
    const int round_bf16 = a.round_bf16;
    const float* bias = a.bias;
    const float renorm_floor = a.renorm_floor, scale = a.scale;
    float s[PER], c[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = j * 32 + lane;
        float x = -INFINITY;
        if (e < E)
            x = BF16_IN ? __bfloat162float(static_cast<const __nv_bfloat16*>(logits)[t * ld + e]) : static_cast<const float*>(logits)[t * ld + e];
        s[j] = x;
        mx = fmaxf(mx, x);
    }
    if (softmax) {
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            s[j] = (j * 32 + lane < E) ? expf(s[j] - mx) : 0.0f;
            sum += s[j];
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
        for (int j = 0; j < PER; ++j) s[j] = __fdiv_rn(s[j], sum);
    } else {
#pragma unroll
        for (int j = 0; j < PER; ++j) s[j] = __fdiv_rn(1.0f, 1.0f + expf(-s[j]));
    }
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = j * 32 + lane;
        if (round_bf16) s[j] = __bfloat162float(__float2bfloat16_rn(s[j]));
        c[j] = e < E ? (bias != nullptr ? s[j] + bias[e] : s[j]) : -INFINITY;      // a fp32 bias promotes the sum to fp32
    }
    // group-limited selection: experts of the groups that are not among the topk_group best are masked out
    if (n_group > 1 && topk_group < n_group) {
        const int gs = E / n_group;
        float gscore = -INFINITY;                 // lane g holds the score of group g (n_group <= 32)
        for (int g = 0; g < n_group; ++g) {
            float m1 = -INFINITY, m2 = -INFINITY; // two largest choice values of group g seen by this lane
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                const int e = j * 32 + lane;
                if (e < E && e / gs == g) {
                    if (c[j] > m1) { m2 = m1; m1 = c[j]; } else if (c[j] > m2) m2 = c[j];
                }
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) {
                const float o1 = __shfl_xor_sync(0xffffffffu, m1, o), o2 = __shfl_xor_sync(0xffffffffu, m2, o);
                const float hi = fmaxf(m1, o1), lo = fminf(m1, o1);
                m2 = fmaxf(lo, fmaxf(m2, o2));
                m1 = hi;
            }
            const float sc = bias != nullptr ? m1 + m2 : m1;
            if (lane == g) gscore = sc;
        }
        unsigned keep = 0;                        // bit g set: group g survives
        for (int r = 0; r < topk_group; ++r) {
            float v = gscore;
            int i = lane;
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) argmax_merge(v, i, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, i, o));
            keep |= 1u << i;
            if (lane == i) gscore = -INFINITY;
        }
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int e = j * 32 + lane;
            if (e < E && !((keep >> (e / gs)) & 1u)) c[j] = -INFINITY;
        }
    }
    // k rounds of warp argmax over the choice values
    float wsum = 0.0f, my_w = 0.0f;
    int my_id = 0;
    for (int r = 0; r < topk; ++r) {
        float v = -INFINITY;
        int i = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < PER; ++j) argmax_merge(v, i, c[j], j * 32 + lane);
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) argmax_merge(v, i, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, i, o));
        float w = 0.0f;
#pragma unroll
        for (int j = 0; j < PER; ++j)
            if (j * 32 + lane == i) {
                w = s[j];
                c[j] = -INFINITY;
            }
        w = __shfl_sync(0xffffffffu, w, i & 31);
        wsum += w;
        if (lane == r) {                          // lane r keeps the r-th choice (topk <= 32)
            my_w = w;
            my_id = i;
        }
    }
    float w = my_w;
    if (lane < topk) {
        if (round_bf16) {
            if (renorm) w = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(w, __bfloat162float(__float2bfloat16_rn(fmaxf(wsum, renorm_floor))))));
            if (scale != 1.0f) w = __bfloat162float(__float2bfloat16_rn(w * scale));
        } else {
            if (renorm) w = __fdiv_rn(w, fmaxf(wsum, renorm_floor));
            if (scale != 1.0f) w *= scale;
        }
    }
    out_weight = w;
    out_id = my_id;
}

}  // namespace kbn
