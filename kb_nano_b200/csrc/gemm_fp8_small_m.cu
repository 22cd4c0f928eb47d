// Block-scaled FP8 GEMM for decode-sized batches (M <= 16 rows of A), the Fp8Linear call of a decode step
// (tasks/baseline/L1/fp8_linear.py:371-450 with M = running sequences).
//
// With so few rows the problem is a weight stream: 2*M flop per weight byte.  The 128-row tcgen05 tile
// kernels give it at most 148 CTAs of one tile each and spend most of their time filling and draining a
// pipeline; here the weights go straight from global memory into registers, 16 weight rows x 128 K-bytes per
// warp and step, with every warp of the GPU streaming at once:
//
//   * the weight rows are the M dimension of mma.sync.m16n8k32 (e4m3 x e4m3 -> fp32), the tokens its N
//     dimension (8 per instruction, two instructions' worth for 9..16 tokens) -- the roles of A and B are
//     swapped, so no tensor-core work is spent on padding rows;
//   * a dot product does not care about the order of K: lane (g, t) loads 16 contiguous bytes of weight row
//     g (and g + 8) at K offset 16*t of each 64-byte half block and the same 16 bytes of its token's row, and
//     both operands use that same permutation of K, so every load is a full 16-byte vector and no shared
//     memory or ldmatrix is needed;
//   * one CTA owns 16 weight rows; its 8 warps split the K-blocks, scale each 128-K partial sum by
//     sa[token, kb] * sw[row / 128, kb] in fp32 (any scales, power of two or not), and add their results in
//     warp order through shared memory.
//
// Algorithmic bytes: N*K of weights + M*K of activations + 2*M*N out; HBM-bound.  Measured on B200 (event-timed, L2
// flushed): 16-18 us for N=4096, K=7168 and M <= 8, the same as the cluster split-K form of the tcgen05 kernel on
// power-of-two scales and half the time of the fp32-scale tcgen05 kernel (32 us), which is the one it replaces.
#include "common.cuh"

namespace kbn {

__device__ __forceinline__ void mma_e4m3_m16n8k32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                                  uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int kSmallMWarps = 8;

// NT: token blocks of 8 (1: M <= 8, 2: M <= 16).
template <int NT>
__global__ void __launch_bounds__(32 * kSmallMWarps)
fp8_gemm_small_m_kernel(const uint8_t* __restrict__ A, const float* __restrict__ sa, int64_t sa_row, int64_t sa_grp,
                        const uint8_t* __restrict__ W, const float* __restrict__ sw, const __nv_bfloat16* __restrict__ bias,
                        __nv_bfloat16* __restrict__ C, int64_t ldc, int M, int N, int K) {
    __shared__ float red[kSmallMWarps][NT * 4][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16;
    const int r0 = n0 + g, r1 = r0 + 8;
    const int KB = (K + 127) >> 7;
    const uint8_t* w0p = W + (int64_t)min(r0, N - 1) * K;
    const uint8_t* w1p = W + (int64_t)min(r1, N - 1) * K;
    const float* swp = sw + (int64_t)(n0 >> 7) * KB;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;

    // The warp's K-blocks (warp, warp + 8, ...) are taken kBatch at a time: all 4 * kBatch weight vectors of a batch
    // are requested before the first is used (256 bytes per lane in flight; a batch of 8 costs a resident CTA per SM
    // and is slower); the activation vectors are fetched as they are needed (they are shared by all CTAs and stay
    // in L1 / L2).
    constexpr int kBatch = 4;
    for (int kb0 = warp; kb0 < KB; kb0 += kSmallMWarps * kBatch) {
        uint4 w0[kBatch][2], w1[kBatch][2];
#pragma unroll
        for (int u = 0; u < kBatch; ++u)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int koff = (kb0 + u * kSmallMWarps) * 128 + h * 64 + t * 16;   // K is a multiple of 16: inside or outside
                const bool in = koff < K;
                w0[u][h] = in ? __ldcs(reinterpret_cast<const uint4*>(w0p + koff)) : zero;
                w1[u][h] = in ? __ldcs(reinterpret_cast<const uint4*>(w1p + koff)) : zero;
            }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int kb = kb0 + u * kSmallMWarps;
            if (kb >= KB) break;
            const float s_w = swp[kb];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int tok_b = nt * 8 + g;
                uint4 x[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int koff = kb * 128 + h * 64 + t * 16;
                    x[h] = (koff < K && tok_b < M) ? __ldg(reinterpret_cast<const uint4*>(A + (int64_t)tok_b * K + koff)) : zero;
                }
                float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    mma_e4m3_m16n8k32(c, w0[u][h].x, w1[u][h].x, w0[u][h].y, w1[u][h].y, x[h].x, x[h].y);
                    mma_e4m3_m16n8k32(c, w0[u][h].z, w1[u][h].z, w0[u][h].w, w1[u][h].w, x[h].z, x[h].w);
                }
                // accumulator columns of this lane are tokens 2t and 2t + 1 of the block
                const int tok = nt * 8 + 2 * t;
                const float s0 = tok < M ? s_w * sa[(int64_t)tok * sa_row + (int64_t)kb * sa_grp] : 0.0f;
                const float s1 = tok + 1 < M ? s_w * sa[(int64_t)(tok + 1) * sa_row + (int64_t)kb * sa_grp] : 0.0f;
                acc[nt][0] = fmaf(c[0], s0, acc[nt][0]);
                acc[nt][1] = fmaf(c[1], s1, acc[nt][1]);
                acc[nt][2] = fmaf(c[2], s0, acc[nt][2]);
                acc[nt][3] = fmaf(c[3], s1, acc[nt][3]);
            }
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[warp][nt * 4 + i][lane] = acc[nt][i];
    __syncthreads();
    // NT*4*32 sums, added in warp order; thread (v, lane) of the first NT*4 warps' worth of threads takes one
    for (int idx = threadIdx.x; idx < NT * 4 * 32; idx += blockDim.x) {
        const int v = idx >> 5, l = idx & 31;
        float sum = 0.0f;
#pragma unroll
        for (int w = 0; w < kSmallMWarps; ++w) sum += red[w][v][l];
        const int nt = v >> 2, i = v & 3;
        const int row = n0 + (l >> 2) + ((i & 2) ? 8 : 0);          // weight row = output column
        const int tok = nt * 8 + 2 * (l & 3) + (i & 1);
        if (row < N && tok < M) C[(int64_t)tok * ldc + row] = __float2bfloat16_rn(bias != nullptr ? sum + __bfloat162float(bias[row]) : sum);
    }
}

// Dense fp32-scale GEMM for M <= 16: returns KBN_OK after launching, or a negative code.
int fp8_gemm_small_m(const void* A, const float* sa, int64_t sa_row, int64_t sa_grp, const void* B, const float* sb, const void* bias,
                     void* C, int64_t ldc, int64_t M, int64_t N, int64_t K, cudaStream_t st) {
    KBN_REQUIRE(M >= 1 && M <= 16 && N >= 1 && K >= 16 && K % 16 == 0, KBN_ERR_ARG, "fp8 gemm (small M): M=%lld N=%lld K=%lld", (long long)M,
                (long long)N, (long long)K);
    KBN_REQUIRE(aligned16(A) && aligned16(B), KBN_ERR_ARG, "fp8 gemm (small M): A and B must be 16-byte aligned");
    KBN_REQUIRE(N < (1ll << 31) - 16 && K < (1ll << 31) - 128, KBN_ERR_ARG, "fp8 gemm (small M): too large");
    const unsigned blocks = (unsigned)((N + 15) / 16);
    const auto* a = static_cast<const uint8_t*>(A);
    const auto* w = static_cast<const uint8_t*>(B);
    auto* c = static_cast<__nv_bfloat16*>(C);
    const auto* b = static_cast<const __nv_bfloat16*>(bias);
    if (M <= 8)
        fp8_gemm_small_m_kernel<1><<<blocks, 32 * kSmallMWarps, 0, st>>>(a, sa, sa_row, sa_grp, w, sb, b, c, ldc, (int)M, (int)N, (int)K);
    else
        fp8_gemm_small_m_kernel<2><<<blocks, 32 * kSmallMWarps, 0, st>>>(a, sa, sa_row, sa_grp, w, sb, b, c, ldc, (int)M, (int)N, (int)K);
    KBN_CHECK_LAUNCH();
    return KBN_OK;
}

}  // namespace kbn
