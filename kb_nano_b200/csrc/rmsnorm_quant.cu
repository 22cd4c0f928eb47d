// Fused (residual-add +) RMSNorm + 1x128 FP8 quantisation: the producer of the activations that the
// FP8 linears consume.  One block per token keeps the whole row in registers, so the row is read
// from HBM once: 2 B in (+2 B residual in, +2 B residual out, +2 B normalised out for the add form) and
// 1 B + 4 B/128 out per element.  HBM-bound.
//
// Arithmetic follows kb-nano's kernel (tasks/baseline/L1/csrc/rmsnorm_quant.cu:22-97,125-204):
//   [add form]  s = fp32(residual) + fp32(x);  residual <- bf16(s);  sum of squares over the unrounded s
//   rms_inv = rsqrtf(sum_sq / H + eps)
//   v = (fp32(r) * rms_inv) * fp32(weight)      with r the bf16 row (rounded sum in the add form)
//   per 128: scale = 2^ceil(log2(max(absmax, 1e-10) / 448)),  q = e4m3(clamp(v / scale, +-448))
//   [add form]  x <- bf16(v)
// Differences that stay inside fp32 rounding noise: the order in which the squares are summed, and the
// scale exponent taken by integer arithmetic instead of log2f/exp2f.
#include "common.cuh"

namespace kbn {

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 8;          // 16-byte vectors per thread: rows up to 256*8*8 = 16384 elements

__device__ __forceinline__ float block_sum(float v, float* smem) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float t = lane < (kNormThreads / 32) ? smem[lane] : 0.0f;
#pragma unroll
    for (int o = 4; o >= 1; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return __shfl_sync(0xffffffffu, t, 0);
}

template <bool ADD>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_quant_kernel(__nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ residual,
                     const __nv_bfloat16* __restrict__ weight, int H, int64_t ld_x, int64_t ld_res,
                     uint8_t* __restrict__ q, int64_t ld_q, float* __restrict__ scale, int64_t s_row, int64_t s_grp,
                     float eps) {
    __shared__ float red[kNormThreads / 32];
    const int64_t token = blockIdx.x;
    const int nvec = H >> 3;
    __nv_bfloat16* xr = x + token * ld_x;
    __nv_bfloat16* rr = ADD ? residual + token * ld_res : nullptr;

    uint4 row[kNormMaxVec];             // the bf16 row that is normalised (x, or the rounded sum)
    float sum_sq = 0.0f;
#pragma unroll
    for (int v = 0; v < kNormMaxVec; ++v) {
        const int idx = threadIdx.x + v * kNormThreads;
        row[v] = make_uint4(0, 0, 0, 0);
        if (idx < nvec) {
            const uint4 a = *reinterpret_cast<const uint4*>(xr + idx * 8);
            if (ADD) {
                const uint4 b = *reinterpret_cast<const uint4*>(rr + idx * 8);
                const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
                uint32_t ow[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float lo = bf16_lo(bw[k]) + bf16_lo(aw[k]), hi = bf16_hi(bw[k]) + bf16_hi(aw[k]);
                    sum_sq = fmaf(lo, lo, sum_sq);
                    sum_sq = fmaf(hi, hi, sum_sq);
                    ow[k] = pack_bf16x2(lo, hi);
                }
                row[v] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                *reinterpret_cast<uint4*>(rr + idx * 8) = row[v];
            } else {
                row[v] = a;
                const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float lo = bf16_lo(aw[k]), hi = bf16_hi(aw[k]);
                    sum_sq = fmaf(lo, lo, sum_sq);
                    sum_sq = fmaf(hi, hi, sum_sq);
                }
            }
        }
    }
    const float rms_inv = rsqrtf(block_sum(sum_sq, red) / (float)H + eps);

    const int j = threadIdx.x & 15;
#pragma unroll
    for (int v = 0; v < kNormMaxVec; ++v) {
        const int idx = threadIdx.x + v * kNormThreads;
        // whole warps leave together: idx is warp-uniform up to the lane, and nvec's tail is handled by `live`
        if ((threadIdx.x & ~31) + v * kNormThreads >= nvec) break;
        const bool live = idx < nvec;
        const uint4 wv = live ? __ldg(reinterpret_cast<const uint4*>(weight + idx * 8)) : make_uint4(0, 0, 0, 0);
        const uint32_t rw[4] = {row[v].x, row[v].y, row[v].z, row[v].w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
        float val[8];
        float amax = 0.0f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            val[2 * k] = __fmul_rn(__fmul_rn(bf16_lo(rw[k]), rms_inv), bf16_lo(ww[k]));
            val[2 * k + 1] = __fmul_rn(__fmul_rn(bf16_hi(rw[k]), rms_inv), bf16_hi(ww[k]));
            amax = fmaxf(amax, fmaxf(fabsf(val[2 * k]), fabsf(val[2 * k + 1])));
        }
#pragma unroll
        for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const uint32_t f = ue8m0_scale_field(fmaxf(amax, 1e-10f));
        const float sc = __uint_as_float(f << 23), inv = __uint_as_float((254u - f) << 23);
        if (live) {
            uint2 o;
            o.x = pack_e4m3x2(val[0] * inv, val[1] * inv) | (pack_e4m3x2(val[2] * inv, val[3] * inv) << 16);
            o.y = pack_e4m3x2(val[4] * inv, val[5] * inv) | (pack_e4m3x2(val[6] * inv, val[7] * inv) << 16);
            *reinterpret_cast<uint2*>(q + token * ld_q + idx * 8) = o;
            if (j == 0) scale[token * s_row + (int64_t)(idx >> 4) * s_grp] = sc;
            if (ADD) {
                uint4 n;
                n.x = pack_bf16x2(val[0], val[1]);
                n.y = pack_bf16x2(val[2], val[3]);
                n.z = pack_bf16x2(val[4], val[5]);
                n.w = pack_bf16x2(val[6], val[7]);
                *reinterpret_cast<uint4*>(xr + idx * 8) = n;
            }
        }
    }
}

static int launch_norm(const char* who, bool add, void* x, void* residual, const void* weight, int64_t M, int64_t H,
                       int64_t ld_x, int64_t ld_res, void* q, int64_t ld_q, float* scale, int64_t s_row, int64_t s_grp,
                       float eps, cudaStream_t st) {
    KBN_REQUIRE(M >= 0 && H >= 0, KBN_ERR_ARG, "%s: negative size", who);
    if (M == 0 || H == 0) return KBN_OK;
    KBN_REQUIRE(x && weight && q && scale && (!add || residual), KBN_ERR_ARG, "%s: null pointer", who);
    KBN_REQUIRE(H % 8 == 0 && H <= kNormThreads * kNormMaxVec * 8, KBN_ERR_UNSUPPORTED,
                "%s: hidden size %lld must be a multiple of 8 and at most %d", who, (long long)H, kNormThreads * kNormMaxVec * 8);
    KBN_REQUIRE(ld_x >= H && ld_q >= H && ld_x % 8 == 0 && ld_q % 8 == 0 && (!add || (ld_res >= H && ld_res % 8 == 0)), KBN_ERR_ARG,
                "%s: row strides must be >= H and multiples of 8", who);
    KBN_REQUIRE(aligned16(x) && aligned16(weight) && (!add || aligned16(residual)) && ((reinterpret_cast<uintptr_t>(q) & 7u) == 0),
                KBN_ERR_ARG, "%s: pointers must be 16-byte aligned (q: 8-byte)", who);
    KBN_REQUIRE(M < (1ll << 31), KBN_ERR_ARG, "%s: too many rows", who);
    auto* xb = static_cast<__nv_bfloat16*>(x);
    auto* rb = static_cast<__nv_bfloat16*>(residual);
    const auto* wb = static_cast<const __nv_bfloat16*>(weight);
    if (add)
        rmsnorm_quant_kernel<true><<<(unsigned)M, kNormThreads, 0, st>>>(xb, rb, wb, (int)H, ld_x, ld_res, static_cast<uint8_t*>(q), ld_q,
                                                                         scale, s_row, s_grp, eps);
    else
        rmsnorm_quant_kernel<false><<<(unsigned)M, kNormThreads, 0, st>>>(xb, nullptr, wb, (int)H, ld_x, 0, static_cast<uint8_t*>(q), ld_q,
                                                                          scale, s_row, s_grp, eps);
    KBN_CHECK_LAUNCH();
    return KBN_OK;
}

}  // namespace kbn

extern "C" int kbn_rmsnorm_quant_1x128(const void* x, const void* weight, int64_t M, int64_t H, int64_t ld_x, void* q,
                                       int64_t ld_q, float* scale, int64_t s_row, int64_t s_grp, float eps,
                                       kbn_stream_t stream) {
    return kbn::launch_norm("kbn_rmsnorm_quant_1x128", false, const_cast<void*>(x), nullptr, weight, M, H, ld_x, 0, q, ld_q, scale,
                            s_row, s_grp, eps, static_cast<cudaStream_t>(stream));
}

extern "C" int kbn_add_rmsnorm_quant_1x128(void* x, void* residual, const void* weight, int64_t M, int64_t H, int64_t ld_x,
                                           int64_t ld_res, void* q, int64_t ld_q, float* scale, int64_t s_row, int64_t s_grp,
                                           float eps, kbn_stream_t stream) {
    return kbn::launch_norm("kbn_add_rmsnorm_quant_1x128", true, x, residual, weight, M, H, ld_x, ld_res, q, ld_q, scale, s_row, s_grp,
                            eps, static_cast<cudaStream_t>(stream));
}
