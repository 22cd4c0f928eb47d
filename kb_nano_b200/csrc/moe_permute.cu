// Token permutation around the two grouped GEMMs of the FP8 MoE expert pipeline.
//
//   permute:  quantised rows [T,K] + scales [T,K/128] + topk_ids [T,topk]
//             -> expert-contiguous rows with 128-aligned segments (stable in (token, slot) order),
//                per-row expert ids (-1 = padding) and the destination row of every (token, slot).
//   combine:  out[t] = sum_s w[t,s] * rows[dest[t,s]]  (fp32 accumulation in slot order, bf16 out)
//
// Replaces the ~15 torch launches of kb-nano's _deepgemm_permute / _deepgemm_unpermute_and_reduce
// (tasks/baseline/L2/fused_experts.py:42-136) with three + one kernels, no host sync and no
// allocation: the only scratch is a caller-provided workspace of 4*(T*topk + 2*E + 2) bytes.
// Everything here is HBM/L2-bound byte shuffling; traffic is (K + 4*K/128) bytes read and written
// per (token, slot) for the permute and 2*H*(topk+1) bytes per token for the combine.
#include "common.cuh"

namespace kbn {

constexpr int kAlign = 128;

// Block e ranks, in flat (token, slot) order, the pairs routed to expert e: every thread counts the
// hits in its own contiguous slice of the pairs, one block-wide exclusive scan turns the counts into
// starting ranks, and a second pass over the slice (still in L1) hands the ranks out.
__global__ void __launch_bounds__(256)
moe_rank_kernel(const int32_t* __restrict__ ids, int64_t n_pairs, int32_t* __restrict__ rank,
                int32_t* __restrict__ counts) {
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ int warp_tot[8];
    const int64_t slice = (((n_pairs + 255) >> 8) + 3) & ~int64_t(3);      // multiple of 4: slices start 16-byte aligned
    const int64_t lo = min((int64_t)threadIdx.x * slice, n_pairs), hi = min(lo + slice, n_pairs);
    const bool vec = (reinterpret_cast<uintptr_t>(ids) & 15u) == 0;
    int cnt = 0;
    int64_t i = lo;
    if (vec)
        for (; i + 4 <= hi; i += 4) {
            const int4 v = *reinterpret_cast<const int4*>(ids + i);
            cnt += (v.x == e) + (v.y == e) + (v.z == e) + (v.w == e);
        }
    for (; i < hi; ++i) cnt += ids[i] == e;
    int incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int next = incl - cnt;
    for (int w = 0; w < warp; ++w) next += warp_tot[w];
    if (threadIdx.x == 255) counts[e] = next + cnt;
    if (cnt == 0) return;
    i = lo;
    if (vec)
        for (; i + 4 <= hi; i += 4) {
            const int4 v = *reinterpret_cast<const int4*>(ids + i);
            if (v.x == e) rank[i] = next++;
            if (v.y == e) rank[i + 1] = next++;
            if (v.z == e) rank[i + 2] = next++;
            if (v.w == e) rank[i + 3] = next++;
        }
    for (; i < hi; ++i)
        if (ids[i] == e) rank[i] = next++;
}

// Aligned exclusive scan of the counts (recomputed by every block: E is small) and the per-row
// expert id of the block's slice of rows.
__global__ void __launch_bounds__(256)
moe_offsets_kernel(const int32_t* __restrict__ counts, int E, int32_t* __restrict__ offsets,
                   int32_t* __restrict__ row_expert, int64_t M_cap) {
    extern __shared__ int32_t sm[];        // offsets[E+1], counts[E]
    int32_t* off = sm;
    int32_t* cnt = sm + E + 1;
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = counts[e];
    __syncthreads();
    if (threadIdx.x == 0) {
        int32_t acc = 0;
        for (int e = 0; e < E; ++e) {
            off[e] = acc;
            acc += (cnt[e] + kAlign - 1) / kAlign * kAlign;
        }
        off[E] = acc;
    }
    __syncthreads();
    if (blockIdx.x == 0)
        for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = off[e];
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < M_cap; r += (int64_t)gridDim.x * blockDim.x) {
        int32_t id = -1;
        if (r < off[E]) {
            int lo = 0, hi = E;            // largest e with off[e] <= r
            while (hi - lo > 1) {
                int mid = (lo + hi) >> 1;
                if (off[mid] <= r) lo = mid; else hi = mid;
            }
            if (r - off[lo] < cnt[lo]) id = lo;
        }
        row_expert[r] = id;
    }
}

// One warp per (token, slot): copy the fp8 row and its scales to the destination row.
__global__ void __launch_bounds__(256)
moe_scatter_kernel(const uint8_t* __restrict__ a_q, const float* __restrict__ a_s, const int32_t* __restrict__ ids,
                   const int32_t* __restrict__ rank, const int32_t* __restrict__ offsets, int64_t n_pairs, int topk,
                   int64_t K, int G, int E, uint8_t* __restrict__ a_perm, float* __restrict__ s_perm,
                   int32_t* __restrict__ dest, uint32_t* __restrict__ sf_packed) {
    const int64_t i = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (i >= n_pairs) return;
    const int lane = threadIdx.x & 31;
    const int e = ids[i];
    if (e < 0 || e >= E) {
        if (lane == 0) dest[i] = -1;
        return;
    }
    const int64_t t = i / topk;
    const int64_t d = (int64_t)offsets[e] + rank[i];
    const uint4* src = reinterpret_cast<const uint4*>(a_q + t * K);
    uint4* dst = reinterpret_cast<uint4*>(a_perm + d * K);
    for (int v = lane; v < (int)(K >> 4); v += 32) dst[v] = __ldg(src + v);
    for (int g = lane; g < G; g += 32) {
        const float sc = __ldg(a_s + t * G + g);
        s_perm[d * G + g] = sc;
        // optional second copy in the packed UE8M0 form the block-scaled GEMM reads: word
        // ((row/128)*G + g)*128 + (row%32)*4 + (row%128)/32 holds the exponent byte four times
        if (sf_packed != nullptr)
            sf_packed[((size_t)(d >> 7) * G + g) * 128u + (size_t)(d & 31) * 4u + (size_t)((d & 127) >> 5)] =
                ((__float_as_uint(sc) >> 23) & 0xffu) * 0x01010101u;
    }
    if (lane == 0) dest[i] = (int32_t)d;
}

// out[t, :] = sum_s w[t,s] * rows[dest[t,s], :]; 8 columns (16 bytes) per thread.
template <int TOPK>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ rows, int64_t ld_rows, const int32_t* __restrict__ dest,
                   const float* __restrict__ w, int64_t T, int topk_rt, int64_t H, __nv_bfloat16* __restrict__ out) {
    const int64_t t = blockIdx.y;
    const int64_t c = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= H) return;
    const int topk = TOPK > 0 ? TOPK : topk_rt;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    auto add = [&](int s) {
        const int32_t d = dest[t * topk + s];
        if (d < 0) return;
        const float ws = w[t * topk + s];
        const uint4 v = __ldcs(reinterpret_cast<const uint4*>(rows + (int64_t)d * ld_rows + c));
        acc[0] = fmaf(ws, bf16_lo(v.x), acc[0]); acc[1] = fmaf(ws, bf16_hi(v.x), acc[1]);
        acc[2] = fmaf(ws, bf16_lo(v.y), acc[2]); acc[3] = fmaf(ws, bf16_hi(v.y), acc[3]);
        acc[4] = fmaf(ws, bf16_lo(v.z), acc[4]); acc[5] = fmaf(ws, bf16_hi(v.z), acc[5]);
        acc[6] = fmaf(ws, bf16_lo(v.w), acc[6]); acc[7] = fmaf(ws, bf16_hi(v.w), acc[7]);
    };
    if (TOPK > 0) {
#pragma unroll
        for (int s = 0; s < TOPK; ++s) add(s);
    } else {
        for (int s = 0; s < topk; ++s) add(s);
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + t * H + c) = o;
}

}  // namespace kbn

extern "C" int kbn_moe_permute_sf(const void*, const float*, const int32_t*, int64_t, int64_t, int64_t, int64_t, void*, float*, int32_t*,
                                  int32_t*, int64_t, void*, int64_t, void*, kbn_stream_t);

namespace kbn {
// Expert of every (token, slot) pair from the sorted, block-padded pair list of kb-nano's Triton MoE path:
// position i of sorted_ids belongs to block i / block_m, whose expert is expert_ids[i / block_m]; entries
// >= n_pairs are padding.  Without a list, block i holds the single pair i.  pair_expert was set to -1 before.
__global__ void moe_pair_experts_kernel(const int32_t* __restrict__ sorted_ids, int64_t n_sorted, const int32_t* __restrict__ expert_ids,
                                        int64_t n_blocks, int32_t block_m, int64_t n_pairs, int32_t* __restrict__ pair_expert) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (sorted_ids == nullptr) {
        if (i < n_pairs && i < n_blocks) pair_expert[i] = expert_ids[i];
        return;
    }
    if (i >= n_sorted || i / block_m >= n_blocks) return;
    const int32_t t = sorted_ids[i];
    if (t >= 0 && t < n_pairs) pair_expert[t] = expert_ids[i / block_m];
}
}  // namespace kbn

extern "C" int kbn_moe_pair_experts(const int32_t* sorted_ids, int64_t n_sorted, const int32_t* expert_ids, int64_t n_blocks,
                                    int64_t block_m, int64_t n_pairs, int32_t* pair_expert, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(n_sorted >= 0 && n_blocks >= 0 && n_pairs >= 0 && block_m > 0 && block_m < (1ll << 31), KBN_ERR_ARG, "kbn_moe_pair_experts: bad sizes");
    if (n_pairs == 0) return KBN_OK;
    KBN_REQUIRE(pair_expert && (n_blocks == 0 || expert_ids), KBN_ERR_ARG, "kbn_moe_pair_experts: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    KBN_CUDA(cudaMemsetAsync(pair_expert, 0xff, (size_t)n_pairs * sizeof(int32_t), st));        // -1: in no block
    const int64_t n = sorted_ids ? n_sorted : n_pairs;
    if (n == 0 || n_blocks == 0) return KBN_OK;
    KBN_REQUIRE((n + 255) / 256 < (1ll << 31), KBN_ERR_ARG, "kbn_moe_pair_experts: too many entries");
    moe_pair_experts_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(sorted_ids, n_sorted, expert_ids, n_blocks, (int32_t)block_m, n_pairs, pair_expert);
    KBN_CHECK_LAUNCH();
    return KBN_OK;
}

extern "C" int64_t kbn_moe_aligned_rows(int64_t T, int64_t topk, int64_t E) {
    int64_t m = T * topk + E * (kbn::kAlign - 1);
    return (m + kbn::kAlign - 1) / kbn::kAlign * kbn::kAlign;
}

extern "C" int64_t kbn_moe_permute_workspace_bytes(int64_t T, int64_t topk, int64_t E) {
    return 4 * (T * topk + 2 * E + 2);
}

extern "C" int kbn_moe_permute(const void* a_q, const float* a_s, const int32_t* topk_ids, int64_t T, int64_t topk,
                               int64_t K, int64_t E, void* a_perm, float* a_s_perm, int32_t* row_expert,
                               int32_t* dest_row, int64_t M_cap, void* workspace, int64_t workspace_bytes,
                               kbn_stream_t stream) {
    return kbn_moe_permute_sf(a_q, a_s, topk_ids, T, topk, K, E, a_perm, a_s_perm, row_expert, dest_row, M_cap, workspace,
                              workspace_bytes, nullptr, stream);
}

extern "C" int kbn_moe_permute_sf(const void* a_q, const float* a_s, const int32_t* topk_ids, int64_t T, int64_t topk,
                                  int64_t K, int64_t E, void* a_perm, float* a_s_perm, int32_t* row_expert,
                                  int32_t* dest_row, int64_t M_cap, void* workspace, int64_t workspace_bytes,
                                  void* a_sf_packed, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(T >= 0 && topk > 0 && K > 0 && E > 0, KBN_ERR_ARG, "kbn_moe_permute: bad sizes");
    KBN_REQUIRE(K % 128 == 0, KBN_ERR_ARG, "kbn_moe_permute: K=%lld must be a multiple of 128", (long long)K);
    KBN_REQUIRE(E <= 4096, KBN_ERR_UNSUPPORTED, "kbn_moe_permute: at most 4096 experts");
    KBN_REQUIRE(M_cap >= kbn_moe_aligned_rows(T, topk, E), KBN_ERR_ARG, "kbn_moe_permute: M_cap=%lld below the aligned row bound %lld",
                (long long)M_cap, (long long)kbn_moe_aligned_rows(T, topk, E));
    KBN_REQUIRE(M_cap < (1ll << 31) && T * topk < (1ll << 31), KBN_ERR_ARG, "kbn_moe_permute: too many rows");
    KBN_REQUIRE(a_perm && a_s_perm && row_expert && dest_row && workspace, KBN_ERR_ARG, "kbn_moe_permute: null pointer");
    KBN_REQUIRE(workspace_bytes >= kbn_moe_permute_workspace_bytes(T, topk, E), KBN_ERR_ARG, "kbn_moe_permute: workspace too small");
    KBN_REQUIRE(aligned16(a_perm) && (T == 0 || aligned16(a_q)), KBN_ERR_ARG, "kbn_moe_permute: rows must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t n_pairs = T * topk;
    int32_t* counts = static_cast<int32_t*>(workspace);
    int32_t* offsets = counts + E;
    int32_t* rank = offsets + E + 1;
    if (n_pairs > 0) KBN_REQUIRE(a_q && a_s && topk_ids, KBN_ERR_ARG, "kbn_moe_permute: null pointer");
    moe_rank_kernel<<<(unsigned)E, 256, 0, st>>>(topk_ids, n_pairs, rank, counts);
    KBN_CHECK_LAUNCH();
    const int off_blocks = (int)((M_cap + 255) / 256 < 64 ? (M_cap + 255) / 256 : 64);
    moe_offsets_kernel<<<off_blocks > 0 ? off_blocks : 1, 256, (size_t)(2 * E + 1) * 4, st>>>(counts, (int)E, offsets, row_expert, M_cap);
    KBN_CHECK_LAUNCH();
    if (n_pairs > 0) {
        moe_scatter_kernel<<<(unsigned)((n_pairs + 7) / 8), 256, 0, st>>>(
            static_cast<const uint8_t*>(a_q), a_s, topk_ids, rank, offsets, n_pairs, (int)topk, K, (int)(K / 128), (int)E,
            static_cast<uint8_t*>(a_perm), a_s_perm, dest_row, static_cast<uint32_t*>(a_sf_packed));
        KBN_CHECK_LAUNCH();
    }
    return KBN_OK;
}

extern "C" int kbn_moe_unpermute_combine(const void* rows, int64_t ld_rows, const int32_t* dest_row, const float* topk_w,
                                         int64_t T, int64_t topk, int64_t H, void* out, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(T >= 0 && topk > 0 && H > 0, KBN_ERR_ARG, "kbn_moe_unpermute_combine: bad sizes");
    if (T == 0) return KBN_OK;
    KBN_REQUIRE(rows && dest_row && topk_w && out, KBN_ERR_ARG, "kbn_moe_unpermute_combine: null pointer");
    KBN_REQUIRE(H % 8 == 0 && ld_rows % 8 == 0 && aligned16(rows) && aligned16(out), KBN_ERR_ARG,
                "kbn_moe_unpermute_combine: H and ld_rows must be multiples of 8 and pointers 16-byte aligned");
    KBN_REQUIRE(T < 65536ll * 32768ll, KBN_ERR_ARG, "kbn_moe_unpermute_combine: too many tokens");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid((unsigned)((H / 8 + 255) / 256), (unsigned)T);
    KBN_REQUIRE(T <= 2147483647ll, KBN_ERR_ARG, "kbn_moe_unpermute_combine: too many tokens");
    const auto* r = static_cast<const __nv_bfloat16*>(rows);
    auto* o = static_cast<__nv_bfloat16*>(out);
    // grid.y is limited to 65535: fold tokens if needed
    if (T > 65535) {
        for (int64_t t0 = 0; t0 < T; t0 += 65535) {
            int64_t tn = T - t0 < 65535 ? T - t0 : 65535;
            dim3 g2(grid.x, (unsigned)tn);
            moe_combine_kernel<0><<<g2, 256, 0, st>>>(r, ld_rows, dest_row + t0 * topk, topk_w + t0 * topk, tn, (int)topk, H, o + t0 * H);
            KBN_CHECK_LAUNCH();
        }
        return KBN_OK;
    }
    if (topk == 8) moe_combine_kernel<8><<<grid, 256, 0, st>>>(r, ld_rows, dest_row, topk_w, T, 8, H, o);
    else if (topk == 2) moe_combine_kernel<2><<<grid, 256, 0, st>>>(r, ld_rows, dest_row, topk_w, T, 2, H, o);
    else moe_combine_kernel<0><<<grid, 256, 0, st>>>(r, ld_rows, dest_row, topk_w, T, (int)topk, H, o);
    KBN_CHECK_LAUNCH();
    return KBN_OK;
}

// ---- permute without any allocation by anyone ---------------------------------------------------
// Some hosts of this library may not call cudaMalloc at the point where they need a permute: code
// running inside a framework that owns all device memory and hands out none for scratch, a real-time
// serving loop that has frozen its memory map, or a plug-in that is only ever given its input and
// output tensors.  For them the three permute kernels can run on scratch that lives in the library
// image itself: a file-scope device array, present on every GPU that loads the library until the
// process exits (about 264 KB).  Limits: T*topk <= 65536 pairs and E <= 1024 experts.
namespace kbn {

constexpr int64_t kStaticPermutePairs = 65536;
constexpr int64_t kStaticPermuteExperts = 1024;
constexpr int64_t kStaticPermuteWords = kStaticPermutePairs + 2 * kStaticPermuteExperts + 2;

static __device__ __align__(256) int32_t g_permute_scratch[kStaticPermuteWords];

// Device address of the array on the current device.  In host code `g_permute_scratch` is only a
// handle for the symbol, not an address a kernel may use, so the address is looked up once per device
// (with that device current) and remembered.
static int static_permute_scratch(int32_t** out) {
    static std::atomic<int32_t*> addr[64];      // host threads that race here store the same value
    int dev = 0;
    KBN_CUDA(cudaGetDevice(&dev));
    KBN_REQUIRE(dev >= 0 && dev < 64, KBN_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    int32_t* p = addr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_permute_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_error("kbn_moe_permute_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return KBN_ERR_CUDA;
        }
        addr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return KBN_OK;
}

}  // namespace kbn

// Same contract and outputs as kbn_moe_permute, minus the workspace arguments.  Calls no cudaMalloc,
// cudaFree or allocating library routine.  The first call on a device looks up the scratch address
// (make that call before any stream capture).  All calls on a device share the one scratch array:
// every word a call reads it has written itself earlier in the same call, so nothing needs clearing,
// but two calls whose kernels overlap on the GPU (different streams) would race on it.
extern "C" int kbn_moe_permute_static(const void* a_q, const float* a_s, const int32_t* topk_ids, int64_t T, int64_t topk,
                                      int64_t K, int64_t E, void* a_perm, float* a_s_perm, int32_t* row_expert,
                                      int32_t* dest_row, int64_t M_cap, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(T >= 0 && topk > 0 && E > 0, KBN_ERR_ARG, "kbn_moe_permute_static: bad sizes");
    KBN_REQUIRE(topk <= kStaticPermutePairs && T <= kStaticPermutePairs / topk && E <= kStaticPermuteExperts, KBN_ERR_UNSUPPORTED,
                "kbn_moe_permute_static: T*topk=%lld (limit %lld) or E=%lld (limit %lld) beyond the built-in scratch; "
                "use kbn_moe_permute with a caller-provided workspace",
                (long long)(T <= kStaticPermutePairs ? T * topk : -1), (long long)kStaticPermutePairs, (long long)E, (long long)kStaticPermuteExperts);
    int32_t* scratch = nullptr;
    int rc = static_permute_scratch(&scratch);
    if (rc != KBN_OK) return rc;
    return kbn_moe_permute(a_q, a_s, topk_ids, T, topk, K, E, a_perm, a_s_perm, row_expert, dest_row, M_cap, scratch,
                           kStaticPermuteWords * 4, stream);
}
