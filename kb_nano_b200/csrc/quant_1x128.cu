// Per-token-group (1x128) FP8 quantisation of bf16 activations.  HBM-bound: 16-byte loads,
// half-warp shuffle absmax on packed bf16x2, power-of-two scale by exponent arithmetic, packed
// e4m3x2 converts and 8-byte stores.  Algorithmic traffic: 2 B in + 1 B out per element and one
// 4 B scale per 128 elements.
#include "quant_common.cuh"

namespace kbn {

// One half-warp per chunk of U consecutive groups of one row; all loads are issued before any use.
// Index arithmetic is 32-bit with a single division per thread (chunk -> row).
template <bool UE8M0, int U>
__global__ void __launch_bounds__(256)
quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint32_t K, int64_t ld_x, uint8_t* __restrict__ q,
                   int64_t ld_q, float* __restrict__ scale, int64_t s_row, int64_t s_grp, float eps,
                   uint32_t G, uint32_t chunks_per_row, uint32_t n_chunks, uint32_t* __restrict__ packed) {
    // the kernel behind this one (the GEMM that reads q) may be scheduled under it, as this one under the kernel before it
    // The kernel behind this one (the GEMM that reads q) may be scheduled under it; it waits for this grid before it
    // reads.  This kernel itself is launched the plain way: started under its own predecessor it was measured slower
    // on small inputs (5.3 against 4.3 us on [512, 7168]) and no faster on large ones.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t j = threadIdx.x & 15u;
    const uint32_t chunk = blockIdx.x * 16u + (threadIdx.x >> 4);
    const bool valid = chunk < n_chunks;
    const uint32_t row = valid ? chunk / chunks_per_row : 0u;
    const uint32_t g0 = (chunk - row * chunks_per_row) * U;
    const __nv_bfloat16* xr = x + (int64_t)row * ld_x;
    uint8_t* qr = q + (int64_t)row * ld_q;

    uint4 v[U];
    bool live[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const uint32_t col = (g0 + u) * 128u + j * 8u;
        live[u] = valid && col < K;
        v[u] = live[u] ? __ldcs(reinterpret_cast<const uint4*>(xr + col)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        GroupScale s = make_scale<UE8M0>(halfwarp_absmax(v[u]), eps);
        if (live[u]) {
            const uint32_t g = g0 + u;
            uint2 o;
            o.x = quant_pair<UE8M0>(v[u].x, s) | (quant_pair<UE8M0>(v[u].y, s) << 16);
            o.y = quant_pair<UE8M0>(v[u].z, s) | (quant_pair<UE8M0>(v[u].w, s) << 16);
            *reinterpret_cast<uint2*>(qr + g * 128u + j * 8u) = o;
            if (j == 0) {
                scale[(int64_t)row * s_row + (int64_t)g * s_grp] = s.scale;
                // optional second copy of the scale in the packed UE8M0 form the block-scaled GEMM reads:
                // word ((row/128)*G + g)*128 + (row%32)*4 + (row%128)/32, exponent byte repeated four times
                if (UE8M0 && packed != nullptr)
                    packed[((size_t)(row >> 7) * G + g) * 128u + (row & 31u) * 4u + ((row & 127u) >> 5)] =
                        ((__float_as_uint(s.scale) >> 23) & 0xffu) * 0x01010101u;
            }
        }
    }
}

// Any K / any alignment: one warp per group, element-wise accesses.
template <bool UE8M0>
__global__ void __launch_bounds__(256)
quant_1x128_generic_kernel(const __nv_bfloat16* __restrict__ x, int64_t M, int64_t K, int64_t ld_x,
                           uint8_t* __restrict__ q, int64_t ld_q, float* __restrict__ scale,
                           int64_t s_row, int64_t s_grp, float eps) {
    const int64_t G = (K + 127) >> 7;
    const int64_t gi = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (gi >= M * G) return;
    const int lane = threadIdx.x & 31;
    const int64_t m = gi / G;
    const int64_t k0 = (gi - m * G) * 128;
    const uint16_t* xr = reinterpret_cast<const uint16_t*>(x) + m * ld_x;
    float val[4];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int64_t k = k0 + lane + 32 * i;
        val[i] = k < K ? __uint_as_float((uint32_t)xr[k] << 16) : 0.0f;
        amax = fmaxf(amax, fabsf(val[i]));
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    GroupScale s = make_scale<UE8M0>(amax, eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int64_t k = k0 + lane + 32 * i;
        if (k < K) {
            float f = UE8M0 ? __fmul_rn(val[i], s.inv)
                            : fminf(fmaxf(__fdiv_rn(val[i], s.scale), -kFp8Max), kFp8Max);
            q[m * ld_q + k] = (uint8_t)(pack_e4m3x2(f, 0.0f) & 0xffu);
        }
    }
    if (lane == 0) scale[m * s_row + (k0 >> 7) * s_grp] = s.scale;
}

}  // namespace kbn

namespace kbn {
static int quant_1x128_impl(const void* x, int64_t M, int64_t K, int64_t ld_x, void* q, int64_t ld_q, float* scale, int64_t s_row,
                            int64_t s_grp, float eps, int ue8m0, void* sf_packed, kbn_stream_t stream);
}

extern "C" int kbn_quant_1x128(const void* x, int64_t M, int64_t K, int64_t ld_x, void* q, int64_t ld_q,
                               float* scale, int64_t s_row, int64_t s_grp, float eps, int ue8m0,
                               kbn_stream_t stream) {
    return kbn::quant_1x128_impl(x, M, K, ld_x, q, ld_q, scale, s_row, s_grp, eps, ue8m0, nullptr, stream);
}

extern "C" int kbn_quant_1x128_sf(const void* x, int64_t M, int64_t K, int64_t ld_x, void* q, int64_t ld_q,
                                  float* scale, int64_t s_row, int64_t s_grp, float eps, void* sf_packed,
                                  kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(sf_packed && aligned16(sf_packed), KBN_ERR_ARG, "kbn_quant_1x128_sf: the packed scale buffer must be 16-byte aligned");
    return quant_1x128_impl(x, M, K, ld_x, q, ld_q, scale, s_row, s_grp, eps, 1, sf_packed, stream);
}

static int kbn::quant_1x128_impl(const void* x, int64_t M, int64_t K, int64_t ld_x, void* q, int64_t ld_q, float* scale, int64_t s_row,
                                 int64_t s_grp, float eps, int ue8m0, void* sf_packed, kbn_stream_t stream) {
    using namespace kbn;
    uint32_t* packed = static_cast<uint32_t*>(sf_packed);
    KBN_REQUIRE(M >= 0 && K >= 0, KBN_ERR_ARG, "kbn_quant_1x128: negative size (M=%lld K=%lld)", (long long)M, (long long)K);
    if (M == 0 || K == 0) return KBN_OK;
    KBN_REQUIRE(x && q && scale, KBN_ERR_ARG, "kbn_quant_1x128: null pointer");
    KBN_REQUIRE(ld_x >= K && ld_q >= K, KBN_ERR_ARG, "kbn_quant_1x128: row stride smaller than K");
    KBN_REQUIRE(eps >= 1e-30f && eps < 1e30f, KBN_ERR_ARG, "kbn_quant_1x128: eps %g outside [1e-30, 1e30)", (double)eps);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t G = (K + 127) / 128, NG = M * G;
    const auto* xb = static_cast<const __nv_bfloat16*>(x);
    auto* qb = static_cast<uint8_t*>(q);
    const bool fast = (K % 8 == 0) && (ld_x % 8 == 0) && (ld_q % 8 == 0) && aligned16(x) && ((reinterpret_cast<uintptr_t>(q) & 7u) == 0);
    if (fast) {
        constexpr int U = 4;
        const int64_t cpr = (G + U - 1) / U, n_chunks = M * cpr;
        KBN_REQUIRE(K < (1ll << 31) && n_chunks < (1ll << 31), KBN_ERR_ARG, "kbn_quant_1x128: more than 2^31 groups");
        const unsigned blocks = (unsigned)((n_chunks + 15) / 16);
        if (ue8m0)
            quant_1x128_kernel<true, U><<<blocks, 256, 0, st>>>(xb, (uint32_t)K, ld_x, qb, ld_q, scale, s_row, s_grp, eps,
                                                                 (uint32_t)G, (uint32_t)cpr, (uint32_t)n_chunks, packed);
        else
            quant_1x128_kernel<false, U><<<blocks, 256, 0, st>>>(xb, (uint32_t)K, ld_x, qb, ld_q, scale, s_row, s_grp, eps,
                                                                  (uint32_t)G, (uint32_t)cpr, (uint32_t)n_chunks, nullptr);
    } else {
        KBN_REQUIRE(!packed, KBN_ERR_ARG, "kbn_quant_1x128_sf: K, the row strides and the pointers must allow 16-byte accesses");
        int64_t blocks = (NG + 7) / 8;
        KBN_REQUIRE(blocks < (1ll << 31), KBN_ERR_ARG, "kbn_quant_1x128: too many groups");
        if (ue8m0)
            quant_1x128_generic_kernel<true><<<(unsigned)blocks, 256, 0, st>>>(xb, M, K, ld_x, qb, ld_q, scale, s_row, s_grp, eps);
        else
            quant_1x128_generic_kernel<false><<<(unsigned)blocks, 256, 0, st>>>(xb, M, K, ld_x, qb, ld_q, scale, s_row, s_grp, eps);
    }
    KBN_CHECK_LAUNCH();
    return KBN_OK;
}
