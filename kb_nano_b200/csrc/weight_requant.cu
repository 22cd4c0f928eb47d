// Load-time re-quantisation of block-scaled FP8 weights to power-of-two (UE8M0) scales, so that a
// checkpoint whose 128x128 block scales are arbitrary fp32 can take the block-scaled tensor-core GEMM.
// Per 128x128 block: w = fp32(w_fp8) * scale;  amax = max|w| clamped at eps;  new_scale =
// 2^ceil(log2(amax/448));  w_fp8 <- e4m3(w / new_scale).  This is what kb-nano does with
// deep_gemm.per_block_cast_to_fp8(use_ue8m0=True) in postprocess_fp8_weights
// (tasks/baseline/L1/fp8_linear.py:453-512, batched form :515-554).  One-off, HBM-bound:
// 1 B in + 1 B out per weight.
#include <cuda_fp16.h>

#include "common.cuh"

namespace kbn {

__device__ __forceinline__ float e4m3_to_f32(uint32_t byte) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)byte, __NV_E4M3);
    return __half2float(__half(h));
}

// grid (ceil(K/128), ceil(N/128), E), 256 threads: thread t owns 64 bytes of row t/2 of the block.
__global__ void __launch_bounds__(256)
requant_ue8m0_kernel(uint8_t* __restrict__ w, float* __restrict__ scale, int64_t N, int64_t K, int NB, int KB, float eps) {
    __shared__ float red[8];
    const int kb = blockIdx.x, nb = blockIdx.y;
    const int64_t e = blockIdx.z;
    const int r = threadIdx.x >> 1, c0 = (threadIdx.x & 1) * 64;
    const int64_t n = (int64_t)nb * 128 + r;
    const int64_t k0 = (int64_t)kb * 128 + c0;
    uint8_t* p = w + (e * N + n) * K + k0;
    float* sp = scale + (e * NB + nb) * KB + kb;
    const float s_old = *sp;
    const bool row_ok = n < N;
    const bool vec = row_ok && (k0 + 64 <= K) && ((reinterpret_cast<uintptr_t>(p) & 15u) == 0);

    float v[64];
    float amax = 0.0f;
    if (vec) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 q = reinterpret_cast<const uint4*>(p)[i];
            const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const float f = __fmul_rn(e4m3_to_f32((words[j] >> (8 * b)) & 0xffu), s_old);
                    v[i * 16 + j * 4 + b] = f;
                    amax = fmaxf(amax, fabsf(f));
                }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
            float f = 0.0f;
            if (row_ok && k0 + i < K) f = __fmul_rn(e4m3_to_f32(p[i]), s_old);
            v[i] = f;
            amax = fmaxf(amax, fabsf(f));
        }
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);

    const uint32_t f = ue8m0_scale_field(fmaxf(amax, eps));
    const float inv = __uint_as_float((254u - f) << 23);
    if (vec) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t words[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float* x = v + i * 16 + j * 4;
                words[j] = pack_e4m3x2(x[0] * inv, x[1] * inv) | (pack_e4m3x2(x[2] * inv, x[3] * inv) << 16);
            }
            reinterpret_cast<uint4*>(p)[i] = make_uint4(words[0], words[1], words[2], words[3]);
        }
    } else if (row_ok) {
#pragma unroll
        for (int i = 0; i < 64; ++i)
            if (k0 + i < K) p[i] = (uint8_t)(pack_e4m3x2(v[i] * inv, 0.0f) & 0xffu);
    }
    __syncthreads();                 // every thread has read the old scale
    if (threadIdx.x == 0) *sp = __uint_as_float(f << 23);
}

}  // namespace kbn

extern "C" int kbn_requant_weights_ue8m0(void* w_fp8, float* scale, int64_t E, int64_t N, int64_t K, float eps,
                                         kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(E >= 0 && N >= 0 && K >= 0, KBN_ERR_ARG, "kbn_requant_weights_ue8m0: negative size");
    if (E == 0 || N == 0 || K == 0) return KBN_OK;
    KBN_REQUIRE(w_fp8 && scale, KBN_ERR_ARG, "kbn_requant_weights_ue8m0: null pointer");
    KBN_REQUIRE(eps >= 1e-30f && eps < 1e30f, KBN_ERR_ARG, "kbn_requant_weights_ue8m0: eps %g outside [1e-30, 1e30)", (double)eps);
    const int64_t NB = (N + 127) / 128, KB = (K + 127) / 128;
    KBN_REQUIRE(NB <= 65535 && E <= 65535 && KB < (1ll << 31), KBN_ERR_ARG, "kbn_requant_weights_ue8m0: too many blocks");
    requant_ue8m0_kernel<<<dim3((unsigned)KB, (unsigned)NB, (unsigned)E), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint8_t*>(w_fp8), scale, N, K, (int)NB, (int)KB, eps);
    KBN_CHECK_LAUNCH();
    return KBN_OK;
}
