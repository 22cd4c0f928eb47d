// Block-scaled FP8 GEMM for sm_100a: dense, expert-contiguous grouped and masked grouped forms
// share one persistent, warp-specialised kernel.
//
//   warp 0      TMA producer: 128x128-byte A and B tiles (SWIZZLE_128B) into a kStages ring
//   warp 1      TMEM allocation + tcgen05.mma issue: one 128x128x128 product per K-block into one
//               of four TMEM accumulators (4 UMMAs of K=32, the first overwriting)
//   warps 2..9  promotion + epilogue: each thread owns one output row and 64 columns; per K-block
//               it reads the partial product from TMEM and does acc += partial * sa[m,kb]*sb[nb,kb]
//               in fp32 registers (weight scales may be arbitrary fp32), then writes bf16.
//
// Tensor-bound roofline: 2*M*N*K flop.  HBM-bound (few rows per expert): every weight byte is read
// once per 128-row block of its expert.  No cluster launch and no multicast: each CTA issues its
// own TMA loads.  Every wait is bounded; on expiry the kernel records a code in a status word,
// raises a CTA-wide abort flag and falls through to the common teardown (TMEM is released).
#include <cuda.h>

#include "gemm_common.cuh"

namespace kbn {

constexpr int kBlockN = 128;
constexpr int kStages = 6;
constexpr int kTileBytes = kBlockM * kBlockK;            // 16 KB per operand tile (fp8)
constexpr int kStageBytes = 2 * kTileBytes;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 32 * (2 + kEpiWarps);
constexpr int kAccBufs = 4;                              // TMEM accumulators in flight (MMA <-> promotion handshake)
constexpr int kTmemCols = kAccBufs * 128;                // all 512 columns: four 128-column fp32 accumulators
constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;

__global__ void __launch_bounds__(kThreads, 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    // SWIZZLE_128B tiles need 1024-byte alignment
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kStages * kStageBytes);
    // bars: [0,kStages) full, [kStages,2kStages) empty, then tmem_full[kAccBufs], tmem_empty[kAccBufs]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 2 * kAccBufs);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = ptx::smem_u32(bars), bar_empty = ptx::smem_u32(bars + kStages);
    const uint32_t bar_tfull = ptx::smem_u32(bars + 2 * kStages), bar_tempty = ptx::smem_u32(bars + 2 * kStages + kAccBufs);
    const uint32_t smem_tiles = ptx::smem_u32(smem);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(bar_full + 8 * s, 1);
            ptx::mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < kAccBufs; ++b) {
            ptx::mbar_init(bar_tfull + 8 * b, 1);
            ptx::mbar_init(bar_tempty + 8 * b, kEpiWarps);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int KB = p.num_k_blocks;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            ptx::prefetch_tensormap(&tmA);
            ptx::prefetch_tensormap(&tmB);
            WaitCtx w{abort_flag, p.status, 1};
            TileWalk walk(p);
            Tile tile;
            uint32_t it = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; ok && walk.get(t, tile); t += gridDim.x) {
                if (!tile.compute) continue;
                const int32_t b_row = tile.expert * p.N + tile.n_blk * kBlockN;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    if (!wait_bar(bar_empty + 8 * s, ph ^ 1u, w)) { ok = false; break; }
                    ptx::mbar_arrive_expect_tx(bar_full + 8 * s, kStageBytes);
                    const uint32_t dst = smem_tiles + s * kStageBytes;
                    ptx::tma_load_2d(dst, &tmA, kb * kBlockK, tile.row0, bar_full + 8 * s);
                    ptx::tma_load_2d(dst + kTileBytes, &tmB, kb * kBlockK, b_row, bar_full + 8 * s);
                }
            }
            if (!ok) {
                // let copies already in flight land before the CTA's shared memory is released
                const long long t0 = clock64();
                while (clock64() - t0 < 400000ll) __nanosleep(1000);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            WaitCtx w{abort_flag, p.status, 2};
            TileWalk walk(p);
            Tile tile;
            uint32_t it = 0;
            constexpr uint32_t idesc = ptx::umma_idesc_e4m3_f32(kBlockM, kBlockN);
            bool ok = true;
            for (int64_t t = blockIdx.x; ok && walk.get(t, tile); t += gridDim.x) {
                if (!tile.compute) continue;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    const uint32_t ab = it % kAccBufs, aph = (it / kAccBufs) & 1u;
                    if (!wait_bar(bar_tempty + 8 * ab, aph ^ 1u, w)) { ok = false; break; }
                    if (!wait_bar(bar_full + 8 * s, ph, w)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint32_t a_addr = smem_tiles + s * kStageBytes;
                    const uint64_t a_desc = ptx::umma_desc_k_sw128(a_addr);
                    const uint64_t b_desc = ptx::umma_desc_k_sw128(a_addr + kTileBytes);
                    const uint32_t d_tmem = tmem_base + ab * kBlockN;
#pragma unroll
                    for (int k = 0; k < kBlockK / 32; ++k) {
                        // advancing 32 bytes along K inside the swizzle atom = +2 in 16-byte units
                        ptx::mma_f8f6f4(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, k > 0 ? 1u : 0u);
                    }
                    ptx::mma_commit(bar_empty + 8 * s);       // smem stage reusable once the MMAs have read it
                    ptx::mma_commit(bar_tfull + 8 * ab);      // partial product ready
                }
            }
        }
    } else {
        // ---------------- promotion + epilogue ----------------
        const int ew = warp - 2;
        const int quarter = warp & 3;            // TMEM lanes this warp may read: 32*quarter ..
        const int half = ew >> 2;                // columns 64*half .. 64*half+63
        const int r_in_tile = quarter * 32 + lane;
        WaitCtx w{abort_flag, p.status, 3};
        TileWalk walk(p);
        Tile tile;
        uint32_t it = 0;
        bool ok = true;
        for (int64_t t = blockIdx.x; ok && walk.get(t, tile); t += gridDim.x) {
            if (!tile.compute) continue;
            const int32_t row = tile.row0 + r_in_tile;
            bool row_ok = row < tile.row_end;
            if (p.mode == kContig && row_ok) row_ok = p.row_expert[row] >= 0;
            const float* sa_ptr;
            if (p.mode == kMasked)
                sa_ptr = p.sa + (int64_t)tile.expert * p.sa_exp + (int64_t)(row - tile.expert * p.max_m) * p.sa_row;
            else
                sa_ptr = p.sa + (int64_t)row * p.sa_row;
            const float* sb_ptr = p.sb + ((int64_t)tile.expert * p.sb_nb + tile.n_blk) * KB;
            float acc[64];
#pragma unroll
            for (int j = 0; j < 64; ++j) acc[j] = 0.0f;
            float sa_next = row_ok ? __ldg(sa_ptr) : 0.0f;
            float sb_next = __ldg(sb_ptr);
            for (int kb = 0; kb < KB; ++kb, ++it) {
                const float sc = sa_next * sb_next;
                if (kb + 1 < KB) {
                    sa_next = row_ok ? __ldg(sa_ptr + (int64_t)(kb + 1) * p.sa_grp) : 0.0f;
                    sb_next = __ldg(sb_ptr + kb + 1);
                }
                const uint32_t ab = it % kAccBufs, aph = (it / kAccBufs) & 1u;
                if (!wait_bar(bar_tfull + 8 * ab, aph, w)) { ok = false; break; }
                ptx::tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + ab * kBlockN + half * 64;
                uint32_t ra[32], rb[32];
                ptx::tmem_ld_32x32(taddr, ra);
                ptx::tmem_ld_32x32(taddr + 32, rb);
                ptx::tmem_ld_wait(ra);
                ptx::tmem_ld_wait(rb);
                // all TMEM reads of this accumulator are complete: hand it back to the MMA warp
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar_tempty + 8 * ab);
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[j] = fmaf(__uint_as_float(ra[j]), sc, acc[j]);
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[32 + j] = fmaf(__uint_as_float(rb[j]), sc, acc[32 + j]);
            }
            if (!ok) break;
            if (row_ok) {
                const int32_t n0 = tile.n_blk * kBlockN + half * 64;
                if (p.bias != nullptr) {
#pragma unroll
                    for (int j = 0; j < 64; ++j)
                        if (n0 + j < p.N) acc[j] += __bfloat162float(p.bias[n0 + j]);
                }
                __nv_bfloat16* crow = p.C + (int64_t)row * p.ldc + n0;
                if (n0 + 64 <= p.N && ((reinterpret_cast<uintptr_t>(crow) & 15u) == 0)) {
#pragma unroll
                    for (int j = 0; j < 64; j += 8) {
                        uint4 v;
                        v.x = pack_bf16x2(acc[j + 0], acc[j + 1]);
                        v.y = pack_bf16x2(acc[j + 2], acc[j + 3]);
                        v.z = pack_bf16x2(acc[j + 4], acc[j + 5]);
                        v.w = pack_bf16x2(acc[j + 6], acc[j + 7]);
                        *reinterpret_cast<uint4*>(crow + j) = v;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 64; ++j)
                        if (n0 + j < p.N) crow[j] = __float2bfloat16_rn(acc[j]);
                }
            }
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- host side ----------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D uint8 tensor [rows, K] with K contiguous; box = 128 bytes x 128 rows, 128-byte swizzle.
static int make_tmap(CUtensorMap* tm, const void* base, int64_t rows, int64_t K, CUtensorMapL2promotion promo) {
    EncodeTiledFn fn = encode_fn();
    KBN_REQUIRE(fn, KBN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K};
    cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)kBlockM};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    KBN_REQUIRE(r == CUDA_SUCCESS, KBN_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld K=%lld)",
                (int)r, (long long)rows, (long long)K);
    return KBN_OK;
}

static int check_device() {
    static int ok[64] = {0};
    int dev = 0;
    KBN_CUDA(cudaGetDevice(&dev));
    KBN_REQUIRE(dev >= 0 && dev < 64, KBN_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    if (!ok[dev]) {
        int major = 0;
        KBN_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        KBN_REQUIRE(major == 10, KBN_ERR_UNSUPPORTED, "kbn_fp8 GEMMs need an sm_100 device (found major %d)", major);
        KBN_CUDA(cudaFuncSetAttribute(fp8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
        ok[dev] = 1;
    }
    return KBN_OK;
}

static int launch_gemm(const void* A, int64_t a_rows, const void* B, int64_t b_rows, GemmParams& p, int64_t max_tiles,
                       cudaStream_t st) {
    int rc = check_device();
    if (rc != KBN_OK) return rc;
    KBN_REQUIRE(aligned16(A) && aligned16(B), KBN_ERR_ARG, "fp8 gemm: A and B must be 16-byte aligned");
    KBN_REQUIRE(p.K % 16 == 0 && p.K > 0, KBN_ERR_ARG, "fp8 gemm: K=%d must be a positive multiple of 16", p.K);
    KBN_REQUIRE(p.N > 0, KBN_ERR_ARG, "fp8 gemm: N must be positive");
    KBN_REQUIRE(a_rows < (1ll << 31) && b_rows < (1ll << 31), KBN_ERR_ARG, "fp8 gemm: more than 2^31 rows");
    CUtensorMap tmA, tmB;
    rc = make_tmap(&tmA, A, a_rows, p.K, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    if (rc != KBN_OK) return rc;
    rc = make_tmap(&tmB, B, b_rows, p.K, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != KBN_OK) return rc;
    rc = gemm_status_ptr(&p.status);
    if (rc != KBN_OK) return rc;
    int64_t grid = sm_count();
    if (max_tiles < grid) grid = max_tiles;
    if (grid <= 0) return KBN_OK;
    fp8_gemm_kernel<<<(unsigned)grid, kThreads, kSmemBytes, st>>>(tmA, tmB, p);
    KBN_CHECK_LAUNCH();
    return KBN_OK;
}

static inline int32_t cdiv32(int64_t a, int64_t b) { return (int32_t)((a + b - 1) / b); }

}  // namespace kbn

namespace kbn {
int fp8_gemm_small_m(const void* A, const float* sa, int64_t sa_row, int64_t sa_grp, const void* B, const float* sb, const void* bias,
                     void* C, int64_t ldc, int64_t M, int64_t N, int64_t K, cudaStream_t st);   // gemm_fp8_small_m.cu
}

extern "C" int kbn_fp8_gemm_nt(const void* A, const float* sa, int64_t sa_row, int64_t sa_grp, const void* B,
                               const float* sb, const void* bias, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                               kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(M >= 0 && N >= 0 && K >= 0, KBN_ERR_ARG, "kbn_fp8_gemm_nt: negative size");
    if (M == 0 || N == 0) return KBN_OK;
    KBN_REQUIRE(A && sa && B && sb && C, KBN_ERR_ARG, "kbn_fp8_gemm_nt: null pointer");
    KBN_REQUIRE(ldc >= N, KBN_ERR_ARG, "kbn_fp8_gemm_nt: ldc < N");
    // decode-sized batches: a weight-streaming kernel instead of 128-row tiles
    if (M <= 16 && K >= 16 && K % 16 == 0 && aligned16(A) && aligned16(B))
        return fp8_gemm_small_m(A, sa, sa_row, sa_grp, B, sb, bias, C, ldc, M, N, K, static_cast<cudaStream_t>(stream));
    GemmParams p{};
    p.sa = sa; p.sa_exp = 0; p.sa_row = sa_row; p.sa_grp = sa_grp; p.sb = sb;
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    p.C = static_cast<__nv_bfloat16*>(C); p.ldc = ldc;
    p.rows_total = (int32_t)M; p.N = (int32_t)N; p.K = (int32_t)K; p.E = 1; p.max_m = 0;
    p.num_m_blocks = cdiv32(M, kBlockM); p.num_n_blocks = cdiv32(N, kBlockN); p.num_k_blocks = cdiv32(K, kBlockK);
    p.sb_nb = cdiv32(N, 128);
    p.mode = kDense;
    return launch_gemm(A, M, B, N, p, (int64_t)p.num_m_blocks * p.num_n_blocks, static_cast<cudaStream_t>(stream));
}

extern "C" int kbn_fp8_grouped_gemm_contig(const void* A, const float* sa, int64_t sa_row, int64_t sa_grp,
                                           const void* B, const float* sb, void* C, int64_t ldc,
                                           const int32_t* row_expert, int64_t M_sum, int64_t N, int64_t K, int64_t E,
                                           kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(M_sum >= 0 && N >= 0 && K >= 0 && E >= 0, KBN_ERR_ARG, "kbn_fp8_grouped_gemm_contig: negative size");
    if (M_sum == 0 || N == 0 || E == 0) return KBN_OK;
    KBN_REQUIRE(A && sa && B && sb && C && row_expert, KBN_ERR_ARG, "kbn_fp8_grouped_gemm_contig: null pointer");
    KBN_REQUIRE(ldc >= N, KBN_ERR_ARG, "kbn_fp8_grouped_gemm_contig: ldc < N");
    KBN_REQUIRE(E * N < (1ll << 31), KBN_ERR_ARG, "kbn_fp8_grouped_gemm_contig: E*N too large");
    GemmParams p{};
    p.sa = sa; p.sa_exp = 0; p.sa_row = sa_row; p.sa_grp = sa_grp; p.sb = sb;
    p.C = static_cast<__nv_bfloat16*>(C); p.ldc = ldc; p.row_expert = row_expert;
    p.rows_total = (int32_t)M_sum; p.N = (int32_t)N; p.K = (int32_t)K; p.E = (int32_t)E; p.max_m = 0;
    p.num_m_blocks = cdiv32(M_sum, kBlockM); p.num_n_blocks = cdiv32(N, kBlockN); p.num_k_blocks = cdiv32(K, kBlockK);
    p.sb_nb = cdiv32(N, 128);
    p.mode = kContig;
    return launch_gemm(A, M_sum, B, E * N, p, (int64_t)p.num_m_blocks * p.num_n_blocks, static_cast<cudaStream_t>(stream));
}

extern "C" int kbn_fp8_grouped_gemm_masked(const void* A, const float* sa, int64_t sa_exp, int64_t sa_row,
                                           int64_t sa_grp, const void* B, const float* sb, void* C,
                                           const int32_t* masked_m, int64_t E, int64_t max_m, int64_t N, int64_t K,
                                           kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(E >= 0 && max_m >= 0 && N >= 0 && K >= 0, KBN_ERR_ARG, "kbn_fp8_grouped_gemm_masked: negative size");
    if (E == 0 || max_m == 0 || N == 0) return KBN_OK;
    KBN_REQUIRE(A && sa && B && sb && C && masked_m, KBN_ERR_ARG, "kbn_fp8_grouped_gemm_masked: null pointer");
    KBN_REQUIRE(E * N < (1ll << 31) && E * max_m < (1ll << 31), KBN_ERR_ARG, "kbn_fp8_grouped_gemm_masked: too large");
    GemmParams p{};
    p.sa = sa; p.sa_exp = sa_exp; p.sa_row = sa_row; p.sa_grp = sa_grp; p.sb = sb;
    p.C = static_cast<__nv_bfloat16*>(C); p.ldc = N; p.masked_m = masked_m;
    p.rows_total = (int32_t)(E * max_m); p.N = (int32_t)N; p.K = (int32_t)K; p.E = (int32_t)E; p.max_m = (int32_t)max_m;
    p.num_m_blocks = 0; p.num_n_blocks = cdiv32(N, kBlockN); p.num_k_blocks = cdiv32(K, kBlockK);
    p.sb_nb = cdiv32(N, 128);
    p.mode = kMasked;
    const int64_t max_tiles = E * (int64_t)cdiv32(max_m, kBlockM) * p.num_n_blocks;
    return launch_gemm(A, E * max_m, B, E * N, p, max_tiles, static_cast<cudaStream_t>(stream));
}

