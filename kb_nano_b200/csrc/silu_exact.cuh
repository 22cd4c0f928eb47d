// Exactly rounded bf16 SiLU for device code: bf16(g / (1 + exp(-g))) as the reference computes it in
// fp32 (tasks/baseline/L1/silu_mul_quant_fp8.py:54-60), from a fast approximation with a per-eight
// doubt test and a 65,536-entry table of exactly rounded results for the doubtful cases.  Shared by
// the stand-alone fused activation kernels and the GEMM epilogue that applies the activation itself.
#pragma once
#include "common.cuh"

namespace kbn {

// Device table of the current device (filled on first use; the fill is enqueued on `st`).
int silu_table_for_stream(cudaStream_t st, const uint16_t** out);

__device__ __forceinline__ float silu_approx(float g) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return g * r;
}

__device__ __forceinline__ uint32_t min_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("min.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Two gates -> packed bf16x2 silu by the fast path; `doubt` collects, for both values at once, whether
// the fp32 result lies within 64 ulps of a bf16 rounding boundary (low 16 bits within 0x40 of 0x8000).
__device__ __forceinline__ uint32_t silu_fast_pair(uint32_t g2, uint32_t& doubt) {
    const float s0 = silu_approx(bf16_lo(g2)), s1 = silu_approx(bf16_hi(g2));
    // low halves of both results side by side; +0x8040 per half maps the doubtful band onto [0, 0x80]
    const uint32_t lo = __byte_perm(__float_as_uint(s0), __float_as_uint(s1), 0x5410);
    const uint32_t z = (lo + 0x80408040u) & 0xff80ff80u;
    doubt |= (z - 0x00010001u) & ~z & 0x80008000u;          // non-zero iff some 16-bit half of z is zero
    return pack_bf16x2(s0, s1);
}

__device__ __forceinline__ uint32_t silu_table_pair(uint32_t g2, const uint16_t* __restrict__ table) {
    return (uint32_t)table[g2 & 0xffffu] | ((uint32_t)table[g2 >> 16] << 16);
}

// Eight gates (one 16-byte load) times eight ups -> four packed bf16x2 y = bf16(bf16(silu(g)) * up).
// One decision per eight values: if any fast result is doubtful, or any gate is below -8 (where the
// approximation's error grows), all eight come from the exactly rounded table instead.
__device__ __forceinline__ void silu_mul_8(const uint4& g, const uint4& u, const uint16_t* __restrict__ table, uint32_t (&y)[4]) {
    uint32_t doubt = 0;
    uint32_t s0 = silu_fast_pair(g.x, doubt), s1 = silu_fast_pair(g.y, doubt);
    uint32_t s2 = silu_fast_pair(g.z, doubt), s3 = silu_fast_pair(g.w, doubt);
    const uint32_t gm = min_bf16x2(min_bf16x2(g.x, g.y), min_bf16x2(g.z, g.w));
    if (doubt != 0u || !(fminf(bf16_lo(gm), bf16_hi(gm)) >= -8.0f)) {
        s0 = silu_table_pair(g.x, table);
        s1 = silu_table_pair(g.y, table);
        s2 = silu_table_pair(g.z, table);
        s3 = silu_table_pair(g.w, table);
    }
    y[0] = mul_bf16x2(s0, u.x);
    y[1] = mul_bf16x2(s1, u.y);
    y[2] = mul_bf16x2(s2, u.z);
    y[3] = mul_bf16x2(s3, u.w);
}

}  // namespace kbn
