// Expert-parallel FP8 MoE layer: tokens stay on their source GPU, experts are split in contiguous
// blocks over the GPUs of one NVSwitch box, and the exchange in both directions is done by this
// file's kernels with plain peer stores over NVLink (no NCCL, no TMA, no multicast).  With power-of-two
// weight scales a layer call is four launches, the last three started with programmatic stream
// serialisation so that each becomes resident while its predecessor still runs:
//
//   dispatch  one CTA per token: its threads first take the token's row slots with remote atomicAdds on the
//             owners' per-expert counters, then quantise the bf16 row 1x128 into shared memory while those
//             atomics are in flight, then one warp per slot stores the fp8 row, its scales (fp32 and packed
//             UE8M0) and a (source, pair) tag straight into the owner's masked-layout buffers [E_local, max_m, H].
//             The last CTA publishes the step number into this rank's flag on every peer (st.release.sys).
//   GEMM1     masked grouped GEMM with SiLU(gate)*up + 1x128 quantisation in its epilogue.  Every CTA polls the
//             dispatch flags of all ranks (ld.acquire.sys, one-second bound, {20, phase, peer} in the status word on
//             expiry) before it reads a row count; tiles come from an atomic counter; every epilogue warp counts
//             its finished tile for the tile's 128-row block.
//   GEMM2     masked grouped GEMM whose producer loads a block's rows once GEMM1 has finished them (the block's
//             counter) and whose epilogue stores every result row into the source rank's [T, topk, H] staging
//             buffer; its CTAs fill the SMs GEMM1's last tiles leave idle.  The last CTA clears the row counts
//             and publishes the step number into the combine flags.
//   sum       polls the combine flags, adds each token's topk rows in slot order with the router weights (the
//             arithmetic of the single-GPU combine) and, in its last block, advances the step counter.
//
// The step number lives in device memory (`epoch`, the number of completed steps; the running step is
// *epoch + 1), so a step takes no argument that changes from call to call and a captured CUDA graph of
// it can be replayed.  Weight scales that are not powers of two take the fp32-scale GEMMs with kernels
// of their own for the wait, the activation and the return of the rows.
//
// This replaces the tensor-parallel all-reduce kb-nano's MoE layers end with
// (tasks/baseline/L1/allreduce.py:37-48 behind tasks/baseline/L2/deepseek_moe.py:301-302).
// Per rank and step the NVLink traffic is at most T*topk*(H + 4*H/128 + 4) bytes out for the
// dispatch and T*topk*2*H bytes in for the combine.
#include <algorithm>
#include <new>

#include "gemm_common.cuh"
#include "moe_route.cuh"
#include "quant_common.cuh"

extern "C" int kbn_fp8_grouped_gemm_masked(const void*, const float*, int64_t, int64_t, int64_t, const void*, const float*,
                                           void*, const int32_t*, int64_t, int64_t, int64_t, int64_t, kbn_stream_t);

extern "C" int kbn_fp8_grouped_gemm_masked_ue8m0(const void*, const void*, const void*, const void*, void*, const int32_t*, int64_t, int64_t,
                                                 int64_t, int64_t, kbn_stream_t);
extern "C" int64_t kbn_packed_sf_rows_bytes(int64_t, int64_t);

namespace kbn {
int silu_mul_quant_masked(const void* in, int64_t E, int64_t max_m, int64_t N2, void* q, float* scale,
                          const int32_t* masked_m, cudaStream_t st, void* packed_sf);   // silu_mul_quant.cu

namespace mx {
int gemm_masked_ue8m0_combine(const void* A, const void* sfa_packed, const void* B, const void* sfb_packed, const int32_t* masked_m,
                              int64_t E, int64_t max_m, int64_t N, int64_t K, const CombineEpilogue& cb, int64_t expected_m,
                              const EpHooks* hooks, cudaStream_t st);   // gemm_fp8_mx.cu
int gemm1_masked_ue8m0_silu(const void* A, const void* sfa_packed, const void* W13, const void* sfb_packed, void* q, float* scale,
                            void* sf_packed, const int32_t* masked_m, int64_t E, int64_t max_m, int64_t I, int64_t K, int64_t expected_m,
                            const EpHooks* hooks, cudaStream_t st);     // gemm_fp8_mx.cu
}

constexpr int kMaxRanks = kMaxPeerRanks;
constexpr long long kFlagWaitCycles = 2000000000ll;   // about a second

struct EpLayout {          // byte offsets inside each rank's symmetric buffer (identical on all ranks)
    int64_t recv_q, recv_s, recv_sf, recv_meta, counters, flags_dispatch, flags_combine, comb, total;
};

struct EpPeers {
    uint8_t* base[kMaxRanks];
};

}  // namespace kbn

struct kbn_ep_ctx {
    int rank, world, device;
    int64_t experts_total, e_local, max_m, hidden, inter, max_tokens, topk;
    kbn::EpLayout lay;
    uint8_t* sym;                      // this rank's symmetric buffer (cudaMalloc)
    kbn::EpPeers peers;                // base pointers of every rank's buffer in this process
    bool attached;
    // local scratch
    __nv_bfloat16* mm1; uint8_t* a2_q; float* a2_s; __nv_bfloat16* mm2;
    uint8_t* sf2;                      // packed UE8M0 scales of the activation between the GEMMs (UE8M0 GEMM path)
    int32_t* done;                     // [4] block-completion counters of dispatch and combine, the step counter, counter of the sum
    float* route_w; int32_t* route_ids; // [max_tokens*topk] router weights and expert ids of the last routed call
    int32_t* hooks;                    // [2 + e_local*max_m/128] tile counters of the two GEMMs, then one counter per 128-row block
    int64_t n_hooks;
    unsigned long long* trace;         // debug builds (-DKBN_TRACE) only: time stamps, else null
    int32_t* status;                   // [4] code, phase, peer, detail
    int32_t* epoch;                    // device word: completed steps
};

namespace kbn {

static inline int64_t up256(int64_t x) { return (x + 255) / 256 * 256; }

static EpLayout make_layout(const kbn_ep_ctx& c) {
    EpLayout l;
    int64_t o = 0;
    l.recv_q = o;          o += up256(c.e_local * c.max_m * c.hidden);
    l.recv_s = o;          o += up256(c.e_local * c.max_m * (c.hidden / 128) * 4);
    l.recv_sf = o;         o += up256(kbn_packed_sf_rows_bytes(c.e_local * c.max_m, c.hidden));
    l.recv_meta = o;       o += up256(c.e_local * c.max_m * 4);
    l.counters = o;        o += up256(c.e_local * 4);
    l.flags_dispatch = o;  o += up256(kMaxRanks * 4);
    l.flags_combine = o;   o += up256(kMaxRanks * 4);
    l.comb = o;            o += up256(c.max_tokens * c.topk * c.hidden * 2);
    l.total = o;
    return l;
}

// Publishes `epoch` to flag slot `rank` of every peer once every block of the grid has passed here.
__device__ __forceinline__ void signal_when_grid_done(int32_t* done, const EpPeers& peers, int64_t flags_off, int rank,
                                                      int world, const int32_t* epoch, int32_t* counters_to_clear, int n_clear) {
    // one system-wide fence per block, by the thread that counts the block: the barrier orders every other thread's
    // peer stores before it
    __syncthreads();
    __shared__ int last;
    if (threadIdx.x == 0) {
        __threadfence_system();
        last = (atomicAdd(done, 1) == (int)(gridDim.x * gridDim.y) - 1);
    }
    __syncthreads();
    if (!last) return;
    if (counters_to_clear) {
        for (int i = threadIdx.x; i < n_clear; i += blockDim.x) counters_to_clear[i] = 0;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        // one fence: acquire side of the count just read, release side of the flags that follow
        __threadfence_system();
        const int32_t step = *epoch + 1;
        for (int r = 0; r < world; ++r)
            asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(reinterpret_cast<int32_t*>(peers.base[r] + flags_off) + rank), "r"(step) : "memory");
        *done = 0;
    }
}

// One CTA per token (one CTA that only signals when the rank has no tokens).  Dynamic shared memory: the quantised
// row [hidden], its scales fp32 [hidden/128], the row slot and the expert of every top-k slot int32 [2 * topk].
// PER > 0: the kernel routes as well -- warp 0 turns the token's router logits into its top-k experts and weights
// (route_token; PER = experts per lane, BF16_IN = logits' dtype) while the other seven warps quantise the row; the
// weights and ids also go to route_w / route_ids for the weighted sum at the end of the layer.  PER == 0: `ids` given.
template <int PER, bool BF16_IN>
__global__ void __launch_bounds__(256)
ep_dispatch_quant_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ ids, const RouteArgs ra,
                         float* __restrict__ route_w, int32_t* __restrict__ route_ids, int T, int topk, int hidden, int e_local,
                         int max_m, int experts_total, EpPeers peers, EpLayout lay, int rank, int world, const int32_t* epoch,
                         int32_t* done, int32_t* status, int32_t* hooks, int n_hooks, unsigned long long* trace) {
    ptx::launch_dependents();
    KBN_TRACE_MARK2(trace, epoch, 0, 0);
    extern __shared__ __align__(16) uint8_t dsm[];
    const int G = hidden >> 7;
    uint8_t* row_q = dsm;
    float* row_s = reinterpret_cast<float*>(dsm + hidden);
    int32_t* pos_s = reinterpret_cast<int32_t*>(row_s + G);
    int32_t* ids_s = pos_s + topk;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // the tile and block counters of this step's two GEMMs start at zero; the GEMMs touch them only after they have
    // seen this grid's flag, which is published after these stores
    if (blockIdx.x == 0)
        for (int i = tid; i < n_hooks; i += blockDim.x) hooks[i] = 0;
    const int t = blockIdx.x;
    if (t < T) {
        // a row slot for slot s of the token: a remote atomicAdd on the owner's per-expert counter, whose round trip
        // overlaps the quantisation below
        auto take_slot = [&](int s, int e) {
            int pos = -1;
            if (e >= 0 && e < experts_total) {
                const int dst = e / e_local, le = e - dst * e_local;
                pos = atomicAdd_system(reinterpret_cast<int32_t*>(peers.base[dst] + lay.counters) + le, 1);
                if (pos >= max_m) {
                    atomicCAS(status, 0, 10);          // an expert received more than max_m rows
                    status[3] = e;
                    pos = -1;
                }
            } else {
                atomicCAS(status, 0, 11);              // expert id out of range
                status[3] = e;
            }
            ids_s[s] = e;
            pos_s[s] = pos;
        };
        constexpr int kFirstQuantWarp = PER > 0 ? 1 : 0;
        if (PER > 0) {
            if (warp == 0) {
                float w;
                int id;
                route_token<(PER > 0 ? PER : 1), BF16_IN>(ra, t, lane, w, id);
                if (lane < topk) {
                    route_w[t * topk + lane] = w;
                    route_ids[t * topk + lane] = id;
                    take_slot(lane, id);
                }
            }
        } else {
            for (int s = tid; s < topk; s += blockDim.x) take_slot(s, ids[t * topk + s]);
        }
        // 1x128 quantisation of the token's row, a half-warp per group, four groups' loads in flight per half-warp
        if (warp >= kFirstQuantWarp) {
            const int nhw = 2 * (8 - kFirstQuantWarp);
            const uint32_t j = tid & 15u;
            const int hw = (tid >> 4) - 2 * kFirstQuantWarp;
            const __nv_bfloat16* xr = x + (int64_t)t * hidden;
            for (int g0 = 0; g0 < G; g0 += 4 * nhw) {
                uint4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int g = g0 + nhw * u + hw;
                    v[u] = g < G ? __ldcs(reinterpret_cast<const uint4*>(xr + g * 128 + j * 8)) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int g = g0 + nhw * u + hw;
                    const GroupScale sc = make_scale<true>(halfwarp_absmax(v[u]), 1e-10f);
                    if (g < G) {
                        uint2 o;
                        o.x = quant_pair<true>(v[u].x, sc) | (quant_pair<true>(v[u].y, sc) << 16);
                        o.y = quant_pair<true>(v[u].z, sc) | (quant_pair<true>(v[u].w, sc) << 16);
                        *reinterpret_cast<uint2*>(row_q + g * 128 + j * 8) = o;
                        if (j == 0) row_s[g] = sc.scale;
                    }
                }
            }
        }
        __syncthreads();
        // one warp per slot: the row, its scales twice (fp32 for the fp32-scale GEMM, packed UE8M0 words for the
        // block-scaled one: word ((row/128)*G + k)*128 + (row%32)*4 + (row%128)/32, exponent byte repeated) and the tag
        for (int s = warp; s < topk; s += (int)(blockDim.x >> 5)) {
            const int pos = pos_s[s];
            if (pos < 0) continue;
            const int e = ids_s[s];
            const int dst = e / e_local, le = e - dst * e_local;
            uint8_t* pb = peers.base[dst];
            const int64_t row = (int64_t)le * max_m + pos;
            const uint4* src = reinterpret_cast<const uint4*>(row_q);
            uint4* dq = reinterpret_cast<uint4*>(pb + lay.recv_q + row * hidden);
            for (int v = lane; v < (hidden >> 4); v += 32) dq[v] = src[v];
            float* ds = reinterpret_cast<float*>(pb + lay.recv_s) + row * G;
            uint32_t* dp = reinterpret_cast<uint32_t*>(pb + lay.recv_sf) + (size_t)(row >> 7) * G * 128 + (row & 31) * 4 + ((row & 127) >> 5);
            for (int k = lane; k < G; k += 32) {
                const float sv = row_s[k];
                ds[k] = sv;
                dp[(size_t)k * 128] = ((__float_as_uint(sv) >> 23) & 0xffu) * 0x01010101u;
            }
            if (lane == 0) reinterpret_cast<int32_t*>(pb + lay.recv_meta)[row] = (rank << 20) | (t * topk + s);
        }
    }
    KBN_TRACE_MARK2(trace, epoch, 0, 1);
    signal_when_grid_done(done, peers, lay.flags_dispatch, rank, world, epoch, nullptr, 0);
    KBN_TRACE_MARK2(trace, epoch, 0, 2);
}

// One block; thread r waits until source r has published the running step (or the bound runs out).  Used on the
// fp32-scale path only; the block-scaled GEMMs poll the flags themselves.
__global__ void ep_wait_kernel(const int32_t* __restrict__ flags, int world, const int32_t* epoch_word, int phase, int32_t* status) {
    const int r = threadIdx.x;
    const int32_t epoch = *epoch_word + 1;
    if (r < world) {
        const long long t0 = clock64();
        while (ptx::ld_acquire_sys(flags + r) != epoch) {
            if (clock64() - t0 > kFlagWaitCycles) {
                if (atomicCAS(status, 0, 20) == 0) {   // timed out waiting for a peer's signal
                    status[1] = phase;
                    status[2] = r;
                }
                break;
            }
            __nanosleep(64);
        }
    }
}

// out[t, :] = sum_s w[t,s] * comb[t*topk + s, :] once every rank's result rows have arrived: 8 columns (16 bytes) per
// thread, blockIdx.y = token, fp32 accumulation in slot order -- the arithmetic of the single-GPU combine.  Every
// block polls the combine flags (bounded); the last block to finish advances the step counter.
template <int TOPK>
__global__ void __launch_bounds__(256)
ep_sum_kernel(const __nv_bfloat16* __restrict__ comb, const float* __restrict__ w, int T, int topk_rt, int H,
              __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ flags, int world, int32_t* epoch_word, int32_t* done,
              int32_t* status, unsigned long long* trace) {
#ifdef KBN_TRACE
    if (trace && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y < 256) trace[4096 * (*epoch_word & 1) + (3 * 256 + blockIdx.y) * 4 + 0] = trace_now();
#endif
    ptx::grid_dependency_wait();
#ifdef KBN_TRACE
    if (trace && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y < 256) trace[4096 * (*epoch_word & 1) + (3 * 256 + blockIdx.y) * 4 + 1] = trace_now();
#endif
    const int32_t epoch = *epoch_word + 1;
    if ((int)threadIdx.x < world) {
        const long long t0 = clock64();
        while (ptx::ld_acquire_sys(flags + threadIdx.x) != epoch) {
            if (clock64() - t0 > kFlagWaitCycles) {
                if (atomicCAS(status, 0, 20) == 0) {
                    status[1] = 2;
                    status[2] = (int32_t)threadIdx.x;
                }
                break;
            }
            __nanosleep(64);
        }
    }
    __syncthreads();
    const int64_t t = blockIdx.y;
    const int64_t c = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    const int topk = TOPK > 0 ? TOPK : topk_rt;
    if (t < T && c < H) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        auto add = [&](int s) {
            const float ws = w[t * topk + s];
            const uint4 v = __ldcs(reinterpret_cast<const uint4*>(comb + (t * topk + s) * (int64_t)H + c));
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
    // every block has read the step counter by the time the last one gets here
    __syncthreads();
#ifdef KBN_TRACE
    if (trace && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y < 256) trace[4096 * (*epoch_word & 1) + (3 * 256 + blockIdx.y) * 4 + 2] = trace_now();
#endif
    if (threadIdx.x == 0 && atomicAdd(done, 1) == (int)(gridDim.x * gridDim.y) - 1) {
        *done = 0;
        *epoch_word = epoch;
    }
}

// Expert outputs back to their sources: blockIdx.y = local expert, whose first counters[le] rows are
// spread over the warps of its gridDim.x blocks; each lane keeps four 16-byte loads in flight.
__global__ void __launch_bounds__(256)
ep_combine_send_kernel(const __nv_bfloat16* __restrict__ mm2, int hidden, int e_local, int max_m, EpPeers peers, EpLayout lay,
                       int rank, int world, const int32_t* epoch, int32_t* done) {
    const int le = blockIdx.y;
    const int lane = threadIdx.x & 31;
    uint8_t* mine = peers.base[rank];
    int32_t* counters = reinterpret_cast<int32_t*>(mine + lay.counters);
    const int cnt = min(counters[le], max_m);
    const int nvec = hidden >> 3;                       // 16-byte vectors per bf16 row
    for (int pos = blockIdx.x * 8 + (threadIdx.x >> 5); pos < cnt; pos += gridDim.x * 8) {
        const int64_t row = (int64_t)le * max_m + pos;
        const int32_t meta = reinterpret_cast<const int32_t*>(mine + lay.recv_meta)[row];
        const int src = meta >> 20, pair = meta & 0xfffff;
        const uint4* s = reinterpret_cast<const uint4*>(mm2 + row * hidden);
        uint4* d = reinterpret_cast<uint4*>(peers.base[src] + lay.comb + (int64_t)pair * hidden * 2);
        int v = lane;
        for (; v + 96 < nvec; v += 128) {
            const uint4 a0 = s[v], a1 = s[v + 32], a2 = s[v + 64], a3 = s[v + 96];
            d[v] = a0; d[v + 32] = a1; d[v + 64] = a2; d[v + 96] = a3;
        }
        for (; v < nvec; v += 32) d[v] = s[v];
    }
    // the last block also zeroes the counters: every block has read them by then, and no peer
    // starts its next dispatch before it has seen this rank's combine signal
    signal_when_grid_done(done, peers, lay.flags_combine, rank, world, epoch, counters, e_local);
}

}  // namespace kbn

extern "C" int kbn_ep_destroy(kbn_ep_ctx* c);

namespace kbn {
static int ep_allocate(kbn_ep_ctx* c) {
    KBN_CUDA(cudaGetDevice(&c->device));
    c->lay = make_layout(*c);
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->sym), (size_t)c->lay.total));
    KBN_CUDA(cudaMemset(c->sym, 0, (size_t)c->lay.total));
    const int64_t rows = c->e_local * c->max_m;
    c->mm1 = nullptr;      // bf16 GEMM outputs of the fp32-scale path only: allocated by the first call that takes it
    c->mm2 = nullptr;
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->a2_q), (size_t)(rows * c->inter)));
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->a2_s), (size_t)(rows * (c->inter / 128) * 4)));
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->sf2), (size_t)kbn_packed_sf_rows_bytes(rows, c->inter)));
    KBN_CUDA(cudaMemset(c->sf2, 0x7f, (size_t)kbn_packed_sf_rows_bytes(rows, c->inter)));
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->done), 16));
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->status), 16));
    KBN_CUDA(cudaMemset(c->done, 0, 16));
    c->epoch = c->done + 2;            // words 0, 1 and 3: block-completion counters; word 2: completed steps
    KBN_CUDA(cudaMemset(c->status, 0, 16));
    c->n_hooks = 2 + c->e_local * ((c->max_m + 127) / 128);
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->hooks), (size_t)c->n_hooks * 4));
    KBN_CUDA(cudaMemset(c->hooks, 0, (size_t)c->n_hooks * 4));
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->route_w), (size_t)(c->max_tokens * c->topk) * 4));
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->route_ids), (size_t)(c->max_tokens * c->topk) * 4));
#ifdef KBN_TRACE
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->trace), 2 * 4 * 256 * 4 * 8));
    KBN_CUDA(cudaMemset(c->trace, 0, 2 * 4 * 256 * 4 * 8));
#endif
    KBN_CUDA(cudaDeviceSynchronize());
    return KBN_OK;
}
}  // namespace kbn

#ifdef KBN_TRACE
extern "C" int kbn_debug_trace(kbn_ep_ctx* c, unsigned long long* host_out) {
    using namespace kbn;
    KBN_CUDA(cudaDeviceSynchronize());
    KBN_CUDA(cudaMemcpy(host_out, c->trace, 2 * 4 * 256 * 4 * 8, cudaMemcpyDeviceToHost));
    return KBN_OK;
}
#endif

extern "C" int kbn_ep_create(int rank, int world, int64_t experts_total, int64_t max_m, int64_t hidden, int64_t inter,
                             int64_t max_tokens, int64_t topk, kbn_ep_ctx** out) {
    using namespace kbn;
    KBN_REQUIRE(out, KBN_ERR_ARG, "kbn_ep_create: null out pointer");
    KBN_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, KBN_ERR_ARG, "kbn_ep_create: bad rank/world %d/%d", rank, world);
    KBN_REQUIRE(experts_total > 0 && experts_total % world == 0, KBN_ERR_ARG, "kbn_ep_create: experts (%lld) must divide evenly over %d ranks",
                (long long)experts_total, world);
    KBN_REQUIRE(hidden % 128 == 0 && inter % 128 == 0 && hidden > 0 && inter > 0, KBN_ERR_ARG, "kbn_ep_create: hidden and inter must be multiples of 128");
    KBN_REQUIRE(max_m > 0 && max_tokens > 0 && topk > 0 && max_tokens < (1 << 20) && topk < (1 << 20) && max_tokens * topk < (1 << 20), KBN_ERR_ARG,
                "kbn_ep_create: bad max_m/max_tokens/topk");
    KBN_REQUIRE(hidden + 4 * (hidden / 128) + 8 * topk <= 48 * 1024, KBN_ERR_UNSUPPORTED, "kbn_ep_create: hidden=%lld too large for the dispatch kernel",
                (long long)hidden);
    kbn_ep_ctx* c = new (std::nothrow) kbn_ep_ctx();
    KBN_REQUIRE(c, KBN_ERR_CUDA, "kbn_ep_create: out of host memory");
    c->rank = rank; c->world = world;
    c->experts_total = experts_total; c->e_local = experts_total / world; c->max_m = max_m; c->hidden = hidden; c->inter = inter;
    c->max_tokens = max_tokens; c->topk = topk; c->attached = false;
    for (int r = 0; r < kMaxRanks; ++r) c->peers.base[r] = nullptr;
    const int rc = ep_allocate(c);
    if (rc != KBN_OK) {
        kbn_ep_destroy(c);        // frees whatever was allocated before the failure; the error text stays
        return rc;
    }
    c->peers.base[rank] = c->sym;
    if (world == 1) c->attached = true;
    *out = c;
    return KBN_OK;
}

extern "C" int kbn_ep_ipc_handle(kbn_ep_ctx* c, void* out64) {
    using namespace kbn;
    KBN_REQUIRE(c && out64, KBN_ERR_ARG, "kbn_ep_ipc_handle: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    KBN_CUDA(cudaIpcGetMemHandle(&h, c->sym));
    memcpy(out64, &h, 64);
    return KBN_OK;
}

extern "C" int kbn_ep_attach(kbn_ep_ctx* c, const void* handles) {
    using namespace kbn;
    KBN_REQUIRE(c && handles, KBN_ERR_ARG, "kbn_ep_attach: null pointer");
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const uint8_t*>(handles) + 64 * r, 64);
        // An all-zero handle maps that rank onto this rank's own buffer: a rank that never runs, for
        // exercising the bounded waits (its flag is never published) inside one process.
        bool zero = true;
        for (int i = 0; i < 64; ++i) zero = zero && static_cast<const uint8_t*>(handles)[64 * r + i] == 0;
        if (zero) {
            c->peers.base[r] = c->sym;
            continue;
        }
        void* p = nullptr;
        KBN_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        c->peers.base[r] = static_cast<uint8_t*>(p);
    }
    c->attached = true;
    return KBN_OK;
}

extern "C" int64_t kbn_ep_symmetric_bytes(kbn_ep_ctx* c) { return c ? c->lay.total : 0; }

namespace kbn {
// The two block-scaled expert GEMMs as the layer runs them.  in_step: inside a layer call (the GEMMs wait for the dispatch
// flags, GEMM2 clears the row counts and signals the peers); otherwise a repeat of the expert phase on the buffers of the
// last call, for measurement (no waits for peers, no flags, row counts given by the caller and left alone).
static int ep_expert_gemms(kbn_ep_ctx* c, const void* w13, const void* w13_sf_packed, const void* w2, const void* w2_sf_packed,
                           int32_t* counters, int64_t expected_m, bool in_step, cudaStream_t st) {
    const int H = (int)c->hidden, I = (int)c->inter;
    uint8_t* mine = c->sym;
    // GEMM1 with SiLU(gate)*up and the 1x128 quantisation in its epilogue; it waits for every source's rows itself
    EpHooks h1{};
    h1.wait_flags = in_step ? reinterpret_cast<const int32_t*>(mine + c->lay.flags_dispatch) : nullptr;
    h1.epoch = c->epoch;
    h1.ep_status = c->status;
    h1.wait_world = c->world;
    h1.wait_phase = 1;
    h1.sched = nullptr;            // GEMM1's CTAs all start together: round-robin gives every CTA the same share
    h1.tile_done = c->hooks + 2;
    h1.done_signal = 1;
    h1.trace = c->trace;
    int rc = mx::gemm1_masked_ue8m0_silu(mine + c->lay.recv_q, mine + c->lay.recv_sf, w13, w13_sf_packed, c->a2_q, c->a2_s, c->sf2, counters,
                                         c->e_local, c->max_m, I, H, expected_m, &h1, st);
    if (rc != KBN_OK) return rc;
    // GEMM2 whose epilogue writes every result row straight into its source rank's staging buffer (peer stores
    // issued tile by tile while the weights of the next tiles stream in) and signals when the grid is done.  It
    // starts while GEMM1's last tiles run and takes a block's rows once all of GEMM1's epilogue warps (8 per tile,
    // I/128 tiles per block) have counted them.
    CombineEpilogue cb{};
    for (int r = 0; r < c->world; ++r) {
        cb.peer_comb[r] = c->peers.base[r] + c->lay.comb;
        cb.peer_flag[r] = reinterpret_cast<int32_t*>(c->peers.base[r] + c->lay.flags_combine) + c->rank;
    }
    cb.meta = reinterpret_cast<const int32_t*>(mine + c->lay.recv_meta);
    cb.done = c->done + 1;
    cb.counters = counters;
    cb.n_counters = in_step ? (int32_t)c->e_local : 0;
    cb.world = in_step ? c->world : 0;
    cb.epoch = c->epoch;              // the device word
    EpHooks h2 = h1;
    h2.sched = c->hooks + 1;       // GEMM2's CTAs become resident as GEMM1's leave: tiles from a counter
    h2.done_signal = 0;
    h2.done_target = 8 * (I / 128);
    return mx::gemm_masked_ue8m0_combine(c->a2_q, c->sf2, w2, w2_sf_packed, counters, c->e_local, c->max_m, H, I, cb, expected_m, &h2, st);
}
}  // namespace kbn

namespace kbn {
struct EpRouteCall {       // the router logits of a call that routes inside the dispatch kernel
    RouteArgs args;
    int logits_bf16;
};
static int ep_forward(kbn_ep_ctx* c, const void* x_bf16, const int32_t* topk_ids, const float* topk_w, const EpRouteCall* route, int64_t T,
                      const void* w13, const float* w13_s, const void* w2, const float* w2_s, const void* w13_sf_packed,
                      const void* w2_sf_packed, void* out_bf16, kbn_stream_t stream);
}  // namespace kbn

extern "C" int kbn_ep_moe_forward(kbn_ep_ctx* c, const void* x_bf16, const int32_t* topk_ids, const float* topk_w, int64_t T,
                                  const void* w13, const float* w13_s, const void* w2, const float* w2_s,
                                  const void* w13_sf_packed, const void* w2_sf_packed, void* out_bf16, kbn_stream_t stream) {
    using namespace kbn;
    if (T > 0) KBN_REQUIRE(topk_ids && topk_w, KBN_ERR_ARG, "kbn_ep_moe_forward: null routing pointer");
    return ep_forward(c, x_bf16, topk_ids, topk_w, nullptr, T, w13, w13_s, w2, w2_s, w13_sf_packed, w2_sf_packed, out_bf16, stream);
}

extern "C" int kbn_ep_moe_forward_routed(kbn_ep_ctx* c, const void* x_bf16, const void* logits, int logits_bf16, int64_t ld, int64_t T,
                                         int softmax, const float* bias, int64_t n_group, int64_t topk_group, int renormalize,
                                         float renorm_floor, float scale, int round_bf16, const void* w13, const float* w13_s,
                                         const void* w2, const float* w2_s, const void* w13_sf_packed, const void* w2_sf_packed,
                                         void* out_bf16, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(c, KBN_ERR_ARG, "kbn_ep_moe_forward_routed: null context");
    const int64_t E = c->experts_total, topk = c->topk;
    if (T > 0) KBN_REQUIRE(logits, KBN_ERR_ARG, "kbn_ep_moe_forward_routed: null logits");
    KBN_REQUIRE(E <= 32 * kRouteMaxPerLane && topk <= 32 && topk <= E, KBN_ERR_UNSUPPORTED, "kbn_ep_moe_forward_routed: at most %d experts and top-32",
                32 * kRouteMaxPerLane);
    KBN_REQUIRE(ld >= E, KBN_ERR_ARG, "kbn_ep_moe_forward_routed: row stride of the logits below E");
    KBN_REQUIRE(n_group >= 1 && n_group <= 32 && E % n_group == 0 && topk_group >= 1 && topk_group <= n_group && topk <= topk_group * (E / n_group),
                KBN_ERR_ARG, "kbn_ep_moe_forward_routed: n_group=%lld must divide E and be at most 32, topk_group=%lld in [1, n_group], with topk experts left",
                (long long)n_group, (long long)topk_group);
    EpRouteCall rc{RouteArgs{logits, ld, (int)E, softmax, bias, (int)n_group, (int)topk_group, (int)topk, renormalize, renorm_floor, scale, round_bf16},
                   logits_bf16};
    return ep_forward(c, x_bf16, nullptr, nullptr, &rc, T, w13, w13_s, w2, w2_s, w13_sf_packed, w2_sf_packed, out_bf16, stream);
}

extern "C" int kbn_ep_last_routing(kbn_ep_ctx* c, float* out_w, int32_t* out_ids, int64_t T, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(c && out_w && out_ids && T >= 0 && T <= c->max_tokens, KBN_ERR_ARG, "kbn_ep_last_routing: bad arguments");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    KBN_CUDA(cudaMemcpyAsync(out_w, c->route_w, (size_t)(T * c->topk) * 4, cudaMemcpyDeviceToDevice, st));
    KBN_CUDA(cudaMemcpyAsync(out_ids, c->route_ids, (size_t)(T * c->topk) * 4, cudaMemcpyDeviceToDevice, st));
    return KBN_OK;
}

static int kbn::ep_forward(kbn_ep_ctx* c, const void* x_bf16, const int32_t* topk_ids, const float* topk_w, const EpRouteCall* route, int64_t T,
                           const void* w13, const float* w13_s, const void* w2, const float* w2_s, const void* w13_sf_packed,
                           const void* w2_sf_packed, void* out_bf16, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(c, KBN_ERR_ARG, "kbn_ep_moe_forward: null context");
    KBN_REQUIRE(c->attached, KBN_ERR_ARG, "kbn_ep_moe_forward: peers not attached (call kbn_ep_attach)");
    KBN_REQUIRE(T >= 0 && T <= c->max_tokens, KBN_ERR_ARG, "kbn_ep_moe_forward: T=%lld exceeds max_tokens=%lld", (long long)T, (long long)c->max_tokens);
    const bool ue8m0 = w13_sf_packed && w2_sf_packed;
    KBN_REQUIRE(w13 && w2 && (ue8m0 || (w13_s && w2_s)), KBN_ERR_ARG, "kbn_ep_moe_forward: null weight pointer");
    KBN_REQUIRE(!ue8m0 || c->max_m % 128 == 0, KBN_ERR_ARG, "kbn_ep_moe_forward: the UE8M0 path needs max_m to be a multiple of 128");
    if (T > 0) KBN_REQUIRE(x_bf16 && out_bf16, KBN_ERR_ARG, "kbn_ep_moe_forward: null pointer");
    if (route) topk_w = c->route_w;
    if (T > 0) KBN_REQUIRE(aligned16(x_bf16) && aligned16(out_bf16), KBN_ERR_ARG, "kbn_ep_moe_forward: x and out must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int32_t* epoch = c->epoch;
    const int H = (int)c->hidden, I = (int)c->inter, G = H / 128;
    uint8_t* mine = c->sym;
    int32_t* counters = reinterpret_cast<int32_t*>(mine + c->lay.counters);
    const int32_t* flags_dispatch = reinterpret_cast<const int32_t*>(mine + c->lay.flags_dispatch);
    const int32_t* flags_combine = reinterpret_cast<const int32_t*>(mine + c->lay.flags_combine);
    int rc;
    // 1. quantise + dispatch + signal (one block even with no tokens, so that peers are not left waiting)
    const size_t dsmem = (size_t)H + 4 * (size_t)G + 8 * (size_t)c->topk;
    const unsigned dgrid = (unsigned)std::max<int64_t>(T, 1);
    const RouteArgs no_route{};
#define KBN_EP_DISPATCH(P, B, RA, IDS)                                                                                              \
    ep_dispatch_quant_kernel<P, B><<<dgrid, 256, dsmem, st>>>(static_cast<const __nv_bfloat16*>(x_bf16), IDS, RA, c->route_w, c->route_ids, \
                                                              (int)T, (int)c->topk, H, (int)c->e_local, (int)c->max_m, (int)c->experts_total, \
                                                              c->peers, c->lay, c->rank, c->world, epoch, c->done, c->status, c->hooks,      \
                                                              (int)c->n_hooks, c->trace)
    if (!route) {
        KBN_EP_DISPATCH(0, false, no_route, topk_ids);
    } else {
        const int per = (int)((c->experts_total + 31) / 32);
#define KBN_EP_ROUTED(P)                                                              \
    do {                                                                              \
        if (route->logits_bf16) KBN_EP_DISPATCH(P, true, route->args, nullptr);       \
        else KBN_EP_DISPATCH(P, false, route->args, nullptr);                         \
    } while (0)
        if (per <= 1) KBN_EP_ROUTED(1);
        else if (per <= 2) KBN_EP_ROUTED(2);
        else if (per <= 4) KBN_EP_ROUTED(4);
        else if (per <= 8) KBN_EP_ROUTED(8);
        else if (per <= 16) KBN_EP_ROUTED(16);
        else KBN_EP_ROUTED(32);
#undef KBN_EP_ROUTED
    }
#undef KBN_EP_DISPATCH
    KBN_CHECK_LAUNCH();
    // 2. local experts on the received rows.  Rows per expert to expect if every rank brings as many tokens as this one and
    //    the routing is even: it decides the operand order of the masked GEMMs (few rows: weights as the M operand)
    const int64_t expected_m = std::max<int64_t>(1, (T * c->world * c->topk + c->experts_total - 1) / c->experts_total);
    const float* recv_s = reinterpret_cast<const float*>(mine + c->lay.recv_s);
    if (ue8m0) {
        rc = ep_expert_gemms(c, w13, w13_sf_packed, w2, w2_sf_packed, counters, expected_m, true, st);
        if (rc != KBN_OK) return rc;
    } else {
        if (!c->mm1) {
            // Weight scales that are not powers of two (or max_m not a multiple of 128): the GEMMs store bf16 and the
            // wait, the activation and the combine are kernels of their own.  Their two scratch buffers are the size of the
            // receive buffers times 2I and H bf16 and are allocated here, once; not inside a stream capture.
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            KBN_CUDA(cudaStreamIsCapturing(st, &cap));
            KBN_REQUIRE(cap == cudaStreamCaptureStatusNone, KBN_ERR_UNSUPPORTED,
                        "kbn_ep_moe_forward: the first call on the fp32-scale path allocates scratch and cannot be captured");
            const int64_t rows = c->e_local * c->max_m;
            KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->mm1), (size_t)(rows * 2 * I * 2)));
            KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->mm2), (size_t)(rows * H * 2)));
        }
        ep_wait_kernel<<<1, kMaxRanks, 0, st>>>(flags_dispatch, c->world, epoch, 1, c->status);
        KBN_CHECK_LAUNCH();
        rc = kbn_fp8_grouped_gemm_masked(mine + c->lay.recv_q, recv_s, c->max_m * G, G, 1, w13, w13_s, c->mm1, counters, c->e_local, c->max_m, 2 * I, H, stream);
        if (rc != KBN_OK) return rc;
        rc = silu_mul_quant_masked(c->mm1, c->e_local, c->max_m, I, c->a2_q, c->a2_s, counters, st, nullptr);
        if (rc != KBN_OK) return rc;
        rc = kbn_fp8_grouped_gemm_masked(c->a2_q, c->a2_s, c->max_m * (I / 128), I / 128, 1, w2, w2_s, c->mm2, counters, c->e_local, c->max_m, H, I, stream);
        if (rc != KBN_OK) return rc;
        // results back to their sources + signal; blocks per expert: enough to fill the GPU when a rank owns few
        // experts with many rows, never more than the rows need
        const unsigned cs_x = (unsigned)std::min<int64_t>((c->max_m + 7) / 8, std::max<int64_t>(8, (4 * (int64_t)sm_count() + c->e_local - 1) / c->e_local));
        ep_combine_send_kernel<<<dim3(cs_x, (unsigned)c->e_local), 256, 0, st>>>(c->mm2, H, (int)c->e_local, (int)c->max_m, c->peers, c->lay, c->rank,
                                                                                c->world, epoch, c->done + 1);
        KBN_CHECK_LAUNCH();
    }
    // 3. once every rank's rows are back: weighted sum over the topk slots of each local token, in slot order, and the
    //    step counter moves on (the kernel runs with one block when this rank has no tokens)
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)((H / 8 + 255) / 256), (unsigned)std::max<int64_t>(T, 1));
        cfg.blockDim = dim3(256);
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = ue8m0 ? 1 : 0;
        const __nv_bfloat16* comb = reinterpret_cast<const __nv_bfloat16*>(mine + c->lay.comb);
        __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out_bf16);
        const int Ti = (int)T, topk = (int)c->topk, world = c->world;
        int32_t* sum_done = c->done + 3;
        cudaError_t le;
        if (topk == 8) le = cudaLaunchKernelEx(&cfg, ep_sum_kernel<8>, comb, topk_w, Ti, topk, H, o, flags_combine, world, epoch, sum_done, c->status, c->trace);
        else if (topk == 2) le = cudaLaunchKernelEx(&cfg, ep_sum_kernel<2>, comb, topk_w, Ti, topk, H, o, flags_combine, world, epoch, sum_done, c->status, c->trace);
        else le = cudaLaunchKernelEx(&cfg, ep_sum_kernel<0>, comb, topk_w, Ti, topk, H, o, flags_combine, world, epoch, sum_done, c->status, c->trace);
        KBN_CUDA(le);
        KBN_CHECK_LAUNCH();
    }
    return KBN_OK;
}

extern "C" int kbn_ep_status(kbn_ep_ctx* c, int32_t* host_out4, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(c && host_out4, KBN_ERR_ARG, "kbn_ep_status: null pointer");
    KBN_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    KBN_CUDA(cudaMemcpy(host_out4, c->status, 16, cudaMemcpyDeviceToHost));
    return KBN_OK;
}

extern "C" int kbn_ep_expert_phase(kbn_ep_ctx* c, const void* w13, const void* w13_sf_packed, const void* w2, const void* w2_sf_packed,
                                   const int32_t* rows_per_expert, int64_t expected_m, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(c && w13 && w13_sf_packed && w2 && w2_sf_packed && rows_per_expert, KBN_ERR_ARG, "kbn_ep_expert_phase: null pointer");
    KBN_REQUIRE(c->max_m % 128 == 0, KBN_ERR_ARG, "kbn_ep_expert_phase: max_m must be a multiple of 128");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    KBN_CUDA(cudaMemsetAsync(c->hooks, 0, (size_t)c->n_hooks * 4, st));
    return ep_expert_gemms(c, w13, w13_sf_packed, w2, w2_sf_packed, const_cast<int32_t*>(rows_per_expert), expected_m, false, st);
}

extern "C" int kbn_ep_clear_status(kbn_ep_ctx* c, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(c, KBN_ERR_ARG, "kbn_ep_clear_status: null context");
    KBN_CUDA(cudaMemsetAsync(c->status, 0, 16, static_cast<cudaStream_t>(stream)));
    return KBN_OK;
}

extern "C" int kbn_ep_destroy(kbn_ep_ctx* c) {
    if (!c) return KBN_OK;
    cudaDeviceSynchronize();
    for (int r = 0; r < c->world; ++r)
        if (r != c->rank && c->peers.base[r] && c->peers.base[r] != c->sym) cudaIpcCloseMemHandle(c->peers.base[r]);
    cudaFree(c->sym); cudaFree(c->mm1); cudaFree(c->a2_q); cudaFree(c->a2_s);
    cudaFree(c->mm2); cudaFree(c->sf2); cudaFree(c->done); cudaFree(c->status); cudaFree(c->hooks); cudaFree(c->trace); cudaFree(c->route_w); cudaFree(c->route_ids);
    delete c;
    cudaGetLastError();        // a failed release must not surface as the next launch's error
    return KBN_OK;
}
