// Fused SiLU(gate)*up + 1x128 FP8 quantisation (the step between the two MoE/MLP projections).
// HBM-bound: per output group of 128 it reads 256 B of gate and 256 B of up and writes 128 B
// of fp8 plus one fp32 scale.
//
// Exact rounding of silu: the reference rounds g/(1+exp(-g)) (fp32, IEEE ops on a correctly
// rounded exp) to bf16 before the multiply.  There are only 65536 possible gates, so the
// kernel evaluates a 5-instruction approximation (ex2.approx / rcp.approx, error < 2^-20
// relative for g >= -8) and, one decision per eight values, falls back to a device-resident table
// of exactly rounded results when any approximation lands within 64 fp32 ulps of a bf16 rounding
// boundary or any gate is below -8.
// The table is filled once per device by silu_table_kernel (fp64 exp rounded to fp32, then the
// reference's fp32 add and divide).
#include <algorithm>

#include "silu_exact.cuh"

namespace kbn {

constexpr float kFp8MaxS = 448.0f;

__device__ uint16_t g_silu_table[65536];

__global__ void silu_table_kernel(uint16_t* __restrict__ table) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 65536u) return;
    float g = __uint_as_float(i << 16);
    float e = (float)exp(-(double)g);              // correctly rounded fp32 exp(-g)
    float s = __fdiv_rn(g, __fadd_rn(1.0f, e));
    table[i] = __bfloat16_as_ushort(__float2bfloat16_rn(s));
}

__device__ __forceinline__ float halfwarp_absmax4(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    uint32_t m = absmax_bf16x2(absmax_bf16x2(a, b), absmax_bf16x2(c, d));
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) m = absmax_bf16x2(m, __shfl_xor_sync(0xffffffffu, m, o));
    m = abs_bf16x2(m);
    return fmaxf(bf16_lo(m), bf16_hi(m));
}

template <bool UE8M0>
__device__ __forceinline__ uint32_t quant_pair_s(uint32_t w, float scale, float inv) {
    float lo = bf16_lo(w), hi = bf16_hi(w);
    if (UE8M0) {
        lo = __fmul_rn(lo, inv);
        hi = __fmul_rn(hi, inv);
    } else {
        lo = fminf(fmaxf(__fdiv_rn(lo, scale), -kFp8MaxS), kFp8MaxS);
        hi = fminf(fmaxf(__fdiv_rn(hi, scale), -kFp8MaxS), kFp8MaxS);
    }
    return pack_e4m3x2(lo, hi);
}

// One group of 128 outputs held by a half-warp (8 gates + 8 ups per lane): activation, absmax over the
// half-warp, scale, quantise, store.  Both halves of a warp must call this together (full-warp shuffles).
// SMEM: `table` is a shared-memory copy of the exact table and every value is looked up there.
template <bool UE8M0, bool SMEM>
__device__ __forceinline__ void smq_group(bool live, uint32_t row, uint32_t g, uint32_t j, const uint4& gv, const uint4& uv,
                                          uint8_t* __restrict__ q, int64_t ld_q, float* __restrict__ scale, int64_t s_row,
                                          int64_t s_grp, float eps, const uint16_t* __restrict__ table, uint32_t G,
                                          uint32_t* __restrict__ packed) {
    uint32_t y[4];
    if (SMEM) {
        y[0] = mul_bf16x2(silu_table_pair(gv.x, table), uv.x);
        y[1] = mul_bf16x2(silu_table_pair(gv.y, table), uv.y);
        y[2] = mul_bf16x2(silu_table_pair(gv.z, table), uv.z);
        y[3] = mul_bf16x2(silu_table_pair(gv.w, table), uv.w);
    } else {
        silu_mul_8(gv, uv, table, y);
    }
    float a = fmaxf(halfwarp_absmax4(y[0], y[1], y[2], y[3]), eps);
    float sc, inv = 0.0f;
    if (UE8M0) {
        uint32_t f = ue8m0_scale_field(a);
        sc = __uint_as_float(f << 23);
        inv = __uint_as_float((254u - f) << 23);
    } else {
        sc = __fdiv_rn(a, kFp8MaxS);
    }
    if (live) {
        uint2 o;
        o.x = quant_pair_s<UE8M0>(y[0], sc, inv) | (quant_pair_s<UE8M0>(y[1], sc, inv) << 16);
        o.y = quant_pair_s<UE8M0>(y[2], sc, inv) | (quant_pair_s<UE8M0>(y[3], sc, inv) << 16);
        *reinterpret_cast<uint2*>(q + (int64_t)row * ld_q + g * 128u + j * 8u) = o;
        if (j == 0) {
            scale[(int64_t)row * s_row + (int64_t)g * s_grp] = sc;
            // optional second copy of the scale in the packed UE8M0 form the block-scaled GEMM reads:
            // word ((row/128)*G + g)*128 + (row%32)*4 + (row%128)/32, exponent byte repeated four times
            if (UE8M0 && packed != nullptr)
                packed[((size_t)(row >> 7) * G + g) * 128u + (row & 31u) * 4u + ((row & 127u) >> 5)] =
                    ((__float_as_uint(sc) >> 23) & 0xffu) * 0x01010101u;
        }
    }
}

// One chunk = U consecutive groups of one row, handled by a half-warp: all 2*U 16-byte loads are issued
// before the first group is processed.
template <bool UE8M0, int U, bool SMEM = false>
__device__ __forceinline__ void smq_chunk(bool valid, uint32_t row, uint32_t g0, uint32_t j, const __nv_bfloat16* __restrict__ in,
                                          uint32_t N2, int64_t ld_in, uint8_t* __restrict__ q, int64_t ld_q,
                                          float* __restrict__ scale, int64_t s_row, int64_t s_grp, float eps,
                                          const uint16_t* __restrict__ table, uint32_t G, uint32_t* __restrict__ packed = nullptr) {
    const __nv_bfloat16* ir = in + (int64_t)row * ld_in;
    uint4 gv[U], uv[U];
    bool live[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const uint32_t col = (g0 + u) * 128u + j * 8u;
        live[u] = valid && (g0 + u) < G;
        gv[u] = live[u] ? __ldcs(reinterpret_cast<const uint4*>(ir + col)) : make_uint4(0, 0, 0, 0);
        uv[u] = live[u] ? __ldcs(reinterpret_cast<const uint4*>(ir + N2 + col)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
        smq_group<UE8M0, SMEM>(live[u], row, g0 + u, j, gv[u], uv[u], q, ld_q, scale, s_row, s_grp, eps, table, G, packed);
}

// Flat grid: chunk index -> (row, first group) with one 32-bit division per thread.
// ROWS: 0 = every row; 1 = rows with row_info[m] >= 0 (expert-contiguous layout, -1 marks padding);
// 3 = the rows listed in row_info[0..M) (entries < 0 skipped).
template <bool UE8M0, int U, int ROWS>
__global__ void __launch_bounds__(256)
silu_mul_quant_kernel(const __nv_bfloat16* __restrict__ in, uint32_t N2, int64_t ld_in, uint8_t* __restrict__ q,
                      int64_t ld_q, float* __restrict__ scale, int64_t s_row, int64_t s_grp, float eps,
                      const uint16_t* __restrict__ table, const int32_t* __restrict__ row_info, uint32_t G,
                      uint32_t chunks_per_row, uint32_t n_chunks, uint32_t* __restrict__ packed) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // the GEMM behind this kernel may come in under it
    const uint32_t chunk = blockIdx.x * 16u + (threadIdx.x >> 4);
    bool valid = chunk < n_chunks;
    const uint32_t row = valid ? chunk / chunks_per_row : 0u;
    const uint32_t g0 = (chunk - row * chunks_per_row) * U;
    uint32_t out_row = row;
    if (ROWS == 1) valid = valid && row_info[row] >= 0;
    if (ROWS == 3) {                      // `row` indexes a list of rows to process
        const int32_t r = valid ? row_info[row] : -1;
        valid = r >= 0;
        out_row = valid ? (uint32_t)r : 0u;
    }
    smq_chunk<UE8M0, U>(valid, out_row, g0, threadIdx.x & 15u, in, N2, ld_in, q, ld_q, scale, s_row, s_grp, eps, table, G, packed);
}

// One group of 128 outputs held by a QUARTER-warp: lane j owns elements [8j, 8j+8) and [64+8j, 64+8j+8), i.e. two
// 16-byte vectors of gate and two of up (each load instruction of the quarter-warp still covers 128 contiguous
// bytes).  Compared with a half-warp per group, the per-group work -- absmax shuffles, scale arithmetic, scale
// store -- is shared by 16 elements per lane instead of 8.  All values come from the shared-memory table.
// The four quarter-warps of a warp must call this together (full-warp shuffles).
__device__ __forceinline__ void smq_group16(bool live, uint32_t row, uint32_t g, uint32_t j, const uint4 (&gv)[2], const uint4 (&uv)[2],
                                            uint8_t* __restrict__ q, int64_t ld_q, float* __restrict__ scale, int64_t s_row,
                                            int64_t s_grp, float eps, const uint16_t* __restrict__ tab, uint32_t G,
                                            uint32_t* __restrict__ packed) {
    uint32_t y[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        y[4 * h + 0] = mul_bf16x2(silu_table_pair(gv[h].x, tab), uv[h].x);
        y[4 * h + 1] = mul_bf16x2(silu_table_pair(gv[h].y, tab), uv[h].y);
        y[4 * h + 2] = mul_bf16x2(silu_table_pair(gv[h].z, tab), uv[h].z);
        y[4 * h + 3] = mul_bf16x2(silu_table_pair(gv[h].w, tab), uv[h].w);
    }
    uint32_t m = absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(y[0], y[1]), absmax_bf16x2(y[2], y[3])),
                               absmax_bf16x2(absmax_bf16x2(y[4], y[5]), absmax_bf16x2(y[6], y[7])));
#pragma unroll
    for (int o = 4; o >= 1; o >>= 1) m = absmax_bf16x2(m, __shfl_xor_sync(0xffffffffu, m, o));
    m = abs_bf16x2(m);
    const float a = fmaxf(fmaxf(bf16_lo(m), bf16_hi(m)), eps);
    const uint32_t f = ue8m0_scale_field(a);
    const float sc = __uint_as_float(f << 23), inv = __uint_as_float((254u - f) << 23);
    if (live) {
        uint8_t* qrow = q + (int64_t)row * ld_q + g * 128u + j * 8u;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint2 o;
            o.x = quant_pair_s<true>(y[4 * h + 0], sc, inv) | (quant_pair_s<true>(y[4 * h + 1], sc, inv) << 16);
            o.y = quant_pair_s<true>(y[4 * h + 2], sc, inv) | (quant_pair_s<true>(y[4 * h + 3], sc, inv) << 16);
            *reinterpret_cast<uint2*>(qrow + 64 * h) = o;
        }
        if (j == 0) {
            scale[(int64_t)row * s_row + (int64_t)g * s_grp] = sc;
            if (packed != nullptr)
                packed[((size_t)(row >> 7) * G + g) * 128u + (row & 31u) * 4u + ((row & 127u) >> 5)] = f * 0x01010101u;
        }
    }
}

// Large inputs (UE8M0 scales): one persistent block of 1024 threads per SM keeps the whole 128 KB exact table in
// shared memory, so silu costs two shared loads per pair instead of the approximation and its check.  A chunk is
// U consecutive groups of one row and belongs to a quarter-warp.  ROWS as in the flat kernel.
template <int U, int ROWS>
__global__ void __launch_bounds__(1024, 1)
silu_mul_quant_smem_kernel(const __nv_bfloat16* __restrict__ in, uint32_t N2, int64_t ld_in, uint8_t* __restrict__ q,
                           int64_t ld_q, float* __restrict__ scale, int64_t s_row, int64_t s_grp, float eps,
                           const uint16_t* __restrict__ table, const int32_t* __restrict__ row_info, uint32_t G,
                           uint32_t chunks_per_row, uint32_t n_chunks, uint32_t* __restrict__ packed) {
    extern __shared__ __align__(16) uint16_t tab[];
    const uint32_t quarter = (threadIdx.x >> 3) & 3u, j = threadIdx.x & 7u;
    // each block takes one contiguous, equally sized range of chunks (a grid-stride loop would leave
    // most blocks idle during the last, partly filled round)
    const uint32_t lo = (uint32_t)(((uint64_t)n_chunks * blockIdx.x) / gridDim.x);
    const uint32_t hi = (uint32_t)(((uint64_t)n_chunks * (blockIdx.x + 1)) / gridDim.x);
    const uint32_t step = blockDim.x >> 3;
    // Rolling prefetch: the U groups of a chunk sit in registers; as soon as group u of the current chunk
    // has been processed, group u of the warp's next chunk is requested into the same registers, so about
    // (U-1)/U of the register buffer is in flight at any time instead of the buffer draining once per chunk.
    struct Ref { bool valid; uint32_t row, g0; };
    auto ref_of = [&](uint32_t base) -> Ref {
        const uint32_t chunk = base + quarter;
        Ref r;
        r.valid = base < hi && chunk < hi;
        r.row = r.valid ? chunk / chunks_per_row : 0u;
        r.g0 = (chunk - r.row * chunks_per_row) * U;
        if (ROWS != 0) {
            const int32_t info = r.valid ? row_info[r.row] : -1;
            r.valid = r.valid && info >= 0;
            if (ROWS == 3) r.row = r.valid ? (uint32_t)info : 0u;      // list entry = the row to process
        }
        return r;
    };
    uint4 gv[U][2], uv[U][2];
    auto fetch = [&](const Ref& r, int u) {
        const bool live = r.valid && (r.g0 + u) < G;
        const __nv_bfloat16* src = in + (int64_t)r.row * ld_in + (r.g0 + u) * 128u + j * 8u;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            gv[u][h] = live ? __ldcs(reinterpret_cast<const uint4*>(src + 64 * h)) : make_uint4(0, 0, 0, 0);
            uv[u][h] = live ? __ldcs(reinterpret_cast<const uint4*>(src + 64 * h + N2)) : make_uint4(0, 0, 0, 0);
        }
    };
    // The table does not depend on the kernel before this one: it is copied while that kernel may still be running.
    // Every block copies the same 128 KB; each starts at a different offset so that the SMs do not all ask L2 for
    // the same line at the same time.
    const uint32_t rot = (blockIdx.x * 55u) & 8191u;
    for (uint32_t i = threadIdx.x; i < 8192u; i += blockDim.x) {
        const uint32_t k = (i + rot) & 8191u;
        reinterpret_cast<uint4*>(tab)[k] = __ldg(reinterpret_cast<const uint4*>(table) + k);
    }
    pdl_prologue_done();
    uint32_t base = lo + (threadIdx.x >> 5) * 4u;
    Ref cur = ref_of(base);
#pragma unroll
    for (int u = 0; u < U; ++u) fetch(cur, u);
    __syncthreads();
    for (; base < hi; base += step) {
        const Ref nxt = ref_of(base + step);
        const bool any_cur = __any_sync(0xffffffffu, cur.valid);       // warp-uniform: something to do in these four chunks
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (any_cur)
                smq_group16(cur.valid && (cur.g0 + u) < G, cur.row, cur.g0 + u, j, gv[u], uv[u], q, ld_q, scale, s_row, s_grp, eps, tab, G,
                            packed);
            fetch(nxt, u);
        }
        cur = nxt;
    }
}

// Masked layout: blockIdx.y = expert; the blocks of an expert loop over the chunks of its first
// masked_m[e] rows only, so an almost empty buffer costs a handful of blocks, not one per row.
template <bool UE8M0, int U>
__global__ void __launch_bounds__(256)
silu_mul_quant_masked_kernel(const __nv_bfloat16* __restrict__ in, uint32_t N2, int64_t ld_in, uint8_t* __restrict__ q,
                             int64_t ld_q, float* __restrict__ scale, int64_t s_row, int64_t s_grp, float eps,
                             const uint16_t* __restrict__ table, const int32_t* __restrict__ masked_m, uint32_t max_m,
                             uint32_t G, uint32_t chunks_per_row, uint32_t* __restrict__ packed) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // the GEMM behind this kernel may come in under it
    const uint32_t e = blockIdx.y;
    const uint32_t cnt = (uint32_t)min(max(masked_m[e], 0), (int)max_m);
    const uint32_t n = cnt * chunks_per_row;
    const uint32_t half = (threadIdx.x >> 4) & 1u;
    // the loop variable is warp-uniform so that both half-warps stay together for the shuffles
    for (uint32_t base = blockIdx.x * 16u + (threadIdx.x >> 5) * 2u; base < n; base += gridDim.x * 16u) {
        const uint32_t chunk = base + half;
        const bool valid = chunk < n;
        const uint32_t r = valid ? chunk / chunks_per_row : 0u;
        const uint32_t g0 = (chunk - r * chunks_per_row) * U;
        smq_chunk<UE8M0, U>(valid, e * max_m + r, g0, threadIdx.x & 15u, in, N2, ld_in, q, ld_q, scale, s_row, s_grp, eps, table, G, packed);
    }
}

// Every gate through the same device function the main kernel uses (up = 1.0).  Each gate is tested
// alone (the eight values of its group are copies of it), so the per-eight decision is exactly the
// gate's own: whatever neighbours it meets in real data can only send it to the table, never to a
// fast result this probe has not seen.
__global__ void silu_probe_kernel(uint16_t* __restrict__ out, const uint16_t* __restrict__ table) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 65536u) return;
    const uint32_t g2 = i | (i << 16);
    const uint4 g = make_uint4(g2, g2, g2, g2);
    const uint4 one = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
    uint32_t y[4];
    silu_mul_8(g, one, table, y);
    out[i] = (uint16_t)(y[0] & 0xffffu);
}

// Table pointer of the current device; the first call per device enqueues the fill on `st`.
int silu_table_for_stream(cudaStream_t st, const uint16_t** out) {
    static std::atomic<int> ready[64];
    int dev = 0;
    KBN_CUDA(cudaGetDevice(&dev));
    KBN_REQUIRE(dev >= 0 && dev < 64, KBN_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    uint16_t* table = nullptr;
    KBN_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&table), g_silu_table));
    if (!ready[dev].load(std::memory_order_acquire)) {
        // Enqueued on the caller's stream, so the caller's kernel is ordered after it; a second
        // thread racing here merely refills the same values.  The device-wide sync makes the
        // table visible to every other stream before the flag is published.
        silu_table_kernel<<<256, 256, 0, st>>>(table);
        KBN_CHECK_LAUNCH();
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(st, &cap);
        if (cap == cudaStreamCaptureStatusNone) {
            KBN_CUDA(cudaStreamSynchronize(st));
            ready[dev].store(1, std::memory_order_release);
        }
    }
    *out = table;
    return KBN_OK;
}

}  // namespace kbn

namespace kbn {

static int launch_silu_mul_quant(const char* who, const void* in, int64_t M, int64_t N2, int64_t ld_in, void* q, int64_t ld_q,
                                 float* scale, int64_t s_row, int64_t s_grp, float eps, int ue8m0, int rows_mode,
                                 const int32_t* row_info, int64_t max_m, cudaStream_t st, uint32_t* packed = nullptr) {
    KBN_REQUIRE(M >= 0 && N2 >= 0, KBN_ERR_ARG, "%s: negative size", who);
    if (M == 0 || N2 == 0) return KBN_OK;
    KBN_REQUIRE(in && q && scale, KBN_ERR_ARG, "%s: null pointer", who);
    KBN_REQUIRE(rows_mode == 0 || row_info, KBN_ERR_ARG, "%s: null row information", who);
    KBN_REQUIRE(N2 % 128 == 0, KBN_ERR_ARG, "%s: N2=%lld must be a multiple of 128", who, (long long)N2);
    KBN_REQUIRE(ld_in >= 2 * N2 && ld_q >= N2, KBN_ERR_ARG, "%s: row stride too small", who);
    KBN_REQUIRE(ld_in % 8 == 0 && ld_q % 8 == 0 && aligned16(in) && ((reinterpret_cast<uintptr_t>(q) & 7u) == 0),
                KBN_ERR_ARG, "%s: pointers/strides must be 16-byte (in) and 8-byte (q) aligned", who);
    KBN_REQUIRE(eps >= 1e-30f && eps < 1e30f, KBN_ERR_ARG, "%s: eps %g outside [1e-30, 1e30)", who, (double)eps);
    const uint16_t* table = nullptr;
    int rc = silu_table_for_stream(st, &table);
    if (rc != KBN_OK) return rc;
    constexpr int U = 4;
    const int64_t G = N2 / 128, cpr = (G + U - 1) / U, n_chunks = M * cpr;
    KBN_REQUIRE(2 * N2 < (1ll << 31) && n_chunks < (1ll << 31) && max_m < (1ll << 31), KBN_ERR_ARG, "%s: more than 2^31 groups", who);
    const auto* ib = static_cast<const __nv_bfloat16*>(in);
    auto* qb = static_cast<uint8_t*>(q);
    const unsigned nb = (unsigned)((n_chunks + 15) / 16);
    const uint32_t mm = (uint32_t)max_m;
#define KBN_SMQ(UE, RM)                                                                                                   \
    silu_mul_quant_kernel<UE, U, RM><<<nb, 256, 0, st>>>(ib, (uint32_t)N2, ld_in, qb, ld_q, scale, s_row, s_grp, eps, table, \
                                                         row_info, (uint32_t)G, (uint32_t)cpr, (uint32_t)n_chunks, packed)
#define KBN_SMQ_MASKED(UE)                                                                                                \
    silu_mul_quant_masked_kernel<UE, U><<<dim3(masked_x, (unsigned)(M / max_m)), 256, 0, st>>>(                                  \
        ib, (uint32_t)N2, ld_in, qb, ld_q, scale, s_row, s_grp, eps, table, row_info, mm, (uint32_t)G, (uint32_t)cpr, packed)
    // masked layout, blocks per expert: enough to fill the GPU when there are few experts with many rows
    const int64_t n_exp = rows_mode == 2 ? M / max_m : 1;
    const unsigned masked_x = (unsigned)std::min<int64_t>((max_m * cpr + 15) / 16, std::max<int64_t>(4, (8 * (int64_t)sm_count() + n_exp - 1) / std::max<int64_t>(n_exp, 1)));
    // large flat inputs with power-of-two scales: persistent blocks with the exact table in shared memory
    if (rows_mode != 2 && ue8m0 && n_chunks * U >= 32768) {
        constexpr int U2 = 2;                 // groups per quarter-warp: 128 bytes per lane in flight
        const int64_t cpr2 = (G + U2 - 1) / U2, n2c = M * cpr2;
        KBN_REQUIRE(n2c < (1ll << 31), KBN_ERR_ARG, "%s: more than 2^31 groups", who);
        static int attr_set[64] = {0};
        int dev = 0;
        KBN_CUDA(cudaGetDevice(&dev));
        if (dev >= 0 && dev < 64 && !attr_set[dev]) {
            KBN_CUDA(cudaFuncSetAttribute(silu_mul_quant_smem_kernel<U2, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 131072));
            KBN_CUDA(cudaFuncSetAttribute(silu_mul_quant_smem_kernel<U2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 131072));
            KBN_CUDA(cudaFuncSetAttribute(silu_mul_quant_smem_kernel<U2, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 131072));
            attr_set[dev] = 1;
        }
        const unsigned grid = (unsigned)sm_count();
        if (rows_mode == 0)
            KBN_CUDA(launch_pdl(silu_mul_quant_smem_kernel<U2, 0>, dim3(grid), dim3(1024), 131072, st, ib, (uint32_t)N2, ld_in, qb, ld_q, scale, s_row, s_grp,
                                eps, table, row_info, (uint32_t)G, (uint32_t)cpr2, (uint32_t)n2c, packed));
        else if (rows_mode == 1)
            KBN_CUDA(launch_pdl(silu_mul_quant_smem_kernel<U2, 1>, dim3(grid), dim3(1024), 131072, st, ib, (uint32_t)N2, ld_in, qb, ld_q, scale, s_row, s_grp,
                                eps, table, row_info, (uint32_t)G, (uint32_t)cpr2, (uint32_t)n2c, packed));
        else
            KBN_CUDA(launch_pdl(silu_mul_quant_smem_kernel<U2, 3>, dim3(grid), dim3(1024), 131072, st, ib, (uint32_t)N2, ld_in, qb, ld_q, scale, s_row, s_grp,
                                eps, table, row_info, (uint32_t)G, (uint32_t)cpr2, (uint32_t)n2c, packed));
    } else if (rows_mode == 2) {
        KBN_REQUIRE(M / max_m <= 65535, KBN_ERR_ARG, "%s: more than 65535 experts", who);
        if (ue8m0) KBN_SMQ_MASKED(true); else KBN_SMQ_MASKED(false);
    } else if (ue8m0) {
        if (rows_mode == 0) KBN_SMQ(true, 0); else if (rows_mode == 1) KBN_SMQ(true, 1); else KBN_SMQ(true, 3);
    } else {
        if (rows_mode == 0) KBN_SMQ(false, 0); else if (rows_mode == 1) KBN_SMQ(false, 1); else KBN_SMQ(false, 3);
    }
#undef KBN_SMQ
#undef KBN_SMQ_MASKED
    KBN_CHECK_LAUNCH();
    return KBN_OK;
}

// masked layout [E, max_m, 2*N2] -> q [E, max_m, N2], row-major scales [E, max_m, N2/128]
int silu_mul_quant_masked(const void* in, int64_t E, int64_t max_m, int64_t N2, void* q, float* scale,
                          const int32_t* masked_m, cudaStream_t st, void* packed_sf) {
    return launch_silu_mul_quant("silu_mul_quant_masked", in, E * max_m, N2, 2 * N2, q, N2, scale, N2 / 128, 1, 1e-10f, 1, 2,
                                 masked_m, max_m, st, static_cast<uint32_t*>(packed_sf));
}

}  // namespace kbn

extern "C" int kbn_silu_mul_quant_1x128(const void* in, int64_t M, int64_t N2, int64_t ld_in, void* q,
                                        int64_t ld_q, float* scale, int64_t s_row, int64_t s_grp, float eps,
                                        int ue8m0, kbn_stream_t stream) {
    return kbn::launch_silu_mul_quant("kbn_silu_mul_quant_1x128", in, M, N2, ld_in, q, ld_q, scale, s_row, s_grp, eps, ue8m0, 0,
                                      nullptr, 1, static_cast<cudaStream_t>(stream));
}

extern "C" int kbn_silu_mul_quant_1x128_rows(const void* in, int64_t M, int64_t N2, int64_t ld_in, void* q,
                                             int64_t ld_q, float* scale, int64_t s_row, int64_t s_grp, float eps,
                                             int ue8m0, const int32_t* row_expert, kbn_stream_t stream) {
    return kbn::launch_silu_mul_quant("kbn_silu_mul_quant_1x128_rows", in, M, N2, ld_in, q, ld_q, scale, s_row, s_grp, eps, ue8m0, 1,
                                      row_expert, 1, static_cast<cudaStream_t>(stream));
}

extern "C" int kbn_silu_mul_quant_1x128_list(const void* in, int64_t N2, int64_t ld_in, void* q, int64_t ld_q, float* scale,
                                             int64_t s_row, int64_t s_grp, float eps, int ue8m0, const int32_t* row_list,
                                             int64_t n_list, void* sf_packed, kbn_stream_t stream) {
    KBN_REQUIRE(!sf_packed || ue8m0, KBN_ERR_ARG, "kbn_silu_mul_quant_1x128_list: packed scales need ue8m0");
    return kbn::launch_silu_mul_quant("kbn_silu_mul_quant_1x128_list", in, n_list, N2, ld_in, q, ld_q, scale, s_row, s_grp, eps, ue8m0, 3,
                                      row_list, 1, static_cast<cudaStream_t>(stream), static_cast<uint32_t*>(sf_packed));
}

extern "C" int kbn_silu_mul_quant_1x128_masked(const void* in, int64_t E, int64_t max_m, int64_t N2, void* q, float* scale,
                                               const int32_t* masked_m, kbn_stream_t stream) {
    KBN_REQUIRE(E >= 0 && max_m > 0, KBN_ERR_ARG, "kbn_silu_mul_quant_1x128_masked: bad sizes");
    return kbn::silu_mul_quant_masked(in, E, max_m, N2, q, scale, masked_m, static_cast<cudaStream_t>(stream), nullptr);
}

extern "C" int kbn_silu_bf16_table(void* out_u16, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(out_u16, KBN_ERR_ARG, "kbn_silu_bf16_table: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint16_t* table = nullptr;
    int rc = silu_table_for_stream(st, &table);
    if (rc != KBN_OK) return rc;
    silu_probe_kernel<<<256, 256, 0, st>>>(static_cast<uint16_t*>(out_u16), table);
    KBN_CHECK_LAUNCH();
    return KBN_OK;
}
