// Arithmetic of the 1x128 FP8 quantisation, shared by the stand-alone quantiser and by the kernels that quantise
// on the way (the expert-parallel dispatch): scale from the group's absmax, x / scale -> e4m3, half-warp absmax.
#pragma once
#include "common.cuh"

namespace kbn {

constexpr float kFp8Max = 448.0f;

struct GroupScale {
    float scale;   // what is stored
    float inv;     // multiplier used when the scale is a power of two
};

template <bool UE8M0>
__device__ __forceinline__ GroupScale make_scale(float absmax, float eps) {
    GroupScale r;
    float a = fmaxf(absmax, eps);
    if (UE8M0) {
        uint32_t f = ue8m0_scale_field(a);
        r.scale = __uint_as_float(f << 23);
        r.inv = __uint_as_float((254u - f) << 23);
    } else {
        r.scale = __fdiv_rn(a, kFp8Max);
        r.inv = 0.0f;
    }
    return r;
}

// x/scale for one packed bf16 pair -> two e4m3 bytes.  With a power-of-two scale the multiply by
// its reciprocal is the same correctly rounded real number as the reference's division.
template <bool UE8M0>
__device__ __forceinline__ uint32_t quant_pair(uint32_t w, const GroupScale& s) {
    float lo = bf16_lo(w), hi = bf16_hi(w);
    if (UE8M0) {
        lo = __fmul_rn(lo, s.inv);
        hi = __fmul_rn(hi, s.inv);
    } else {
        lo = fminf(fmaxf(__fdiv_rn(lo, s.scale), -kFp8Max), kFp8Max);
        hi = fminf(fmaxf(__fdiv_rn(hi, s.scale), -kFp8Max), kFp8Max);
    }
    return pack_e4m3x2(lo, hi);
}

__device__ __forceinline__ float halfwarp_absmax(uint4 v) {
    uint32_t m = absmax_bf16x2(absmax_bf16x2(v.x, v.y), absmax_bf16x2(v.z, v.w));
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) m = absmax_bf16x2(m, __shfl_xor_sync(0xffffffffu, m, o));
    m = abs_bf16x2(m);
    return fmaxf(bf16_lo(m), bf16_hi(m));
}

}  // namespace kbn
