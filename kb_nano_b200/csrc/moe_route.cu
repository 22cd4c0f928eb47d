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
#include "moe_route.cuh"

namespace kbn {


template <int PER, bool BF16_IN>
__global__ void __launch_bounds__(256)
moe_route_kernel(const RouteArgs a, int64_t T, float* __restrict__ out_w, int32_t* __restrict__ out_ids) {
    const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    const int lane = threadIdx.x & 31;
    float w;
    int id;
    route_token<PER, BF16_IN>(a, t, lane, w, id);
    if (lane < a.topk) {
        out_w[t * a.topk + lane] = w;
        out_ids[t * a.topk + lane] = id;
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
    RouteArgs ra{logits, ld, (int)E, softmax, bias, (int)n_group, (int)topk_group, (int)topk, renormalize, renorm_floor, scale, round_bf16};
#define KBN_ROUTE(P)                                                                              \
    do {                                                                                          \
        if (logits_bf16) moe_route_kernel<P, true><<<blocks, 256, 0, st>>>(ra, T, out_w, out_ids); \
        else moe_route_kernel<P, false><<<blocks, 256, 0, st>>>(ra, T, out_w, out_ids);            \
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
