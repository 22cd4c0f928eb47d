// Expert routing in front of the MoE pipeline: scores (softmax or sigmoid of the router logits), optional
// selection bias, optional group-limited selection, top-k, renormalisation and scaling in one kernel,
// one warp per token.  Stands behind kb-nano's TopKSoftmax (tasks/baseline/L1/topk_softmax.py:37-60; torch
// reference tasks/reference/L1/topk_softmax.py:46-52) and GroupedTopK (tasks/baseline/L1/grouped_topk.py:75-174,
// whose eager path is about ten torch launches per layer and token batch).
//
//   scores   = softmax(logits) or sigmoid(logits), computed in fp32; with round_bf16 the scores and the weight
//              arithmetic are rounded to bf16 step by step, which is what torch does when GroupedTopK is given
//              bf16 logits (it scores in the logits' dtype; TopKSoftmax converts to fp32 first)
//   choice   = scores + bias when a bias is given, else scores
//   groups   = the E experts form n_group contiguous groups; a group's score is the sum of its two largest
//              choice values (with a bias) or its largest one (without); only the topk_group best groups stay
//   top-k    = the k largest choice values among the remaining experts, in descending order (ties: lower index)
//   weights  = the unbiased scores of the chosen experts, divided by their sum when renormalising
//              (TopKSoftmax clamps that sum at 1e-20), times the routed scaling factor
//
// HBM traffic is 4*E bytes per token in and 8*k bytes out; the kernel is bound by the k rounds of warp argmax.
#include "common.cuh"

namespace kbn {

constexpr int kRouteMaxPerLane = 32;      // experts per lane: E <= 1024

__device__ __forceinline__ void argmax_merge(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) {
        v = ov;
        i = oi;
    }
}

// PER = ceil(E / 32) rounded up to a power of two by the host (compile-time unrolling); expert of slot (j, lane)
// is j * 32 + lane.
template <int PER, bool BF16_IN>
__global__ void __launch_bounds__(256)
moe_route_kernel(const void* __restrict__ logits, int64_t ld, int64_t T, int E, int softmax, const float* __restrict__ bias,
                 int n_group, int topk_group, int topk, int renorm, float renorm_floor, float scale, int round_bf16,
                 float* __restrict__ out_w, int32_t* __restrict__ out_ids) {
    const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    const int lane = threadIdx.x & 31;
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
    if (lane < topk) {
        float w = my_w;
        if (round_bf16) {
            if (renorm) w = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(w, __bfloat162float(__float2bfloat16_rn(fmaxf(wsum, renorm_floor))))));
            if (scale != 1.0f) w = __bfloat162float(__float2bfloat16_rn(w * scale));
        } else {
            if (renorm) w = __fdiv_rn(w, fmaxf(wsum, renorm_floor));
            if (scale != 1.0f) w *= scale;
        }
        out_w[t * topk + lane] = w;
        out_ids[t * topk + lane] = my_id;
    }
}

}  // namespace kbn

extern "C" int kbn_moe_route_topk(const void* logits, int logits_bf16, int64_t ld, int64_t T, int64_t E, int softmax, const float* bias,
                                  int64_t n_group, int64_t topk_group, int64_t topk, int renormalize, float renorm_floor, float scale,
                                  int round_bf16, float* out_w, int32_t* out_ids, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(T >= 0 && E > 0 && topk > 0, KBN_ERR_ARG, "kbn_moe_route_topk: bad sizes");
    if (T == 0) return KBN_OK;
    KBN_REQUIRE(logits && out_w && out_ids, KBN_ERR_ARG, "kbn_moe_route_topk: null pointer");
    KBN_REQUIRE(E <= 32 * kRouteMaxPerLane, KBN_ERR_UNSUPPORTED, "kbn_moe_route_topk: at most %d experts", 32 * kRouteMaxPerLane);
    KBN_REQUIRE(topk <= 32 && topk <= E, KBN_ERR_ARG, "kbn_moe_route_topk: topk=%lld must be at most 32 and at most E", (long long)topk);
    KBN_REQUIRE(ld >= E, KBN_ERR_ARG, "kbn_moe_route_topk: row stride below E");
    KBN_REQUIRE(n_group >= 1 && n_group <= 32 && E % n_group == 0 && topk_group >= 1 && topk_group <= n_group, KBN_ERR_ARG,
                "kbn_moe_route_topk: n_group=%lld must divide E and be at most 32, topk_group=%lld in [1, n_group]", (long long)n_group,
                (long long)topk_group);
    KBN_REQUIRE(topk <= topk_group * (E / n_group), KBN_ERR_ARG, "kbn_moe_route_topk: fewer experts in the kept groups than topk");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned blocks = (unsigned)((T + 7) / 8);
    const int per = (int)((E + 31) / 32);
#define KBN_ROUTE(P)                                                                                                               \
    do {                                                                                                                           \
        if (logits_bf16)                                                                                                           \
            moe_route_kernel<P, true><<<blocks, 256, 0, st>>>(logits, ld, T, (int)E, softmax, bias, (int)n_group, (int)topk_group, \
                                                              (int)topk, renormalize, renorm_floor, scale, round_bf16, out_w, out_ids); \
        else                                                                                                                       \
            moe_route_kernel<P, false><<<blocks, 256, 0, st>>>(logits, ld, T, (int)E, softmax, bias, (int)n_group, (int)topk_group, \
                                                               (int)topk, renormalize, renorm_floor, scale, round_bf16, out_w, out_ids); \
    } while (0)
    if (per <= 1) KBN_ROUTE(1);
    else if (per <= 2) KBN_ROUTE(2);
    else if (per <= 4) KBN_ROUTE(4);
    else if (per <= 8) KBN_ROUTE(8);
    else if (per <= 16) KBN_ROUTE(16);
    else KBN_ROUTE(32);
#undef KBN_ROUTE
    KBN_CHECK_LAUNCH();
    return KBN_OK;
}
