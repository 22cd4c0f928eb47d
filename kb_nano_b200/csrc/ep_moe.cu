// Expert-parallel FP8 MoE layer: tokens stay on their source GPU, experts are split in contiguous
// blocks over the GPUs of one NVSwitch box, and the exchange in both directions is done by this
// file's kernels with plain peer stores over NVLink (no NCCL, no TMA, no multicast):
//
//   dispatch  one warp per (token, slot): a remote atomicAdd on the owner's per-expert counter
//             gives the row slot, then the fp8 row, its 1x128 scales and a (source, pair) tag are
//             stored straight into the owner's masked-layout buffers [E_local, max_m, H].
//   signal    the last block of a sender publishes the step number into a per-(source) flag on every peer.
//             The step number lives in device memory (`epoch`, the number of completed steps; the running step is
//             *epoch + 1 and the step's last wait kernel advances it), so a step takes no argument that changes
//             from call to call and a captured CUDA graph of it can be replayed
//             (st.release.sys after a system fence); a one-block kernel on the receiver polls its
//             flags (ld.acquire.sys) with a one-second bound and records {phase, peer} on expiry.
//   experts   masked grouped GEMM1 -> fused SiLU*up+quant (valid rows only) -> masked grouped GEMM2.
//   combine   one warp per received row pushes the bf16 result into the source's [T, topk, H]
//             staging buffer; after the second signal/wait the source adds its topk rows in slot
//             order with the router weights (same arithmetic as the single-GPU combine).
//
// This replaces the tensor-parallel all-reduce kb-nano's MoE layers end with
// (tasks/baseline/L1/allreduce.py:37-48 behind tasks/baseline/L2/deepseek_moe.py:301-302).
// Per rank and step the NVLink traffic is at most T*topk*(H + 4*H/128 + 4) bytes out for the
// dispatch and T*topk*2*H bytes in for the combine.
#include <algorithm>
#include <new>

#include "gemm_common.cuh"

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
                              cudaStream_t st);   // gemm_fp8_mx.cu
int gemm1_masked_ue8m0_silu(const void* A, const void* sfa_packed, const void* W13, const void* sfb_packed, void* q, float* scale,
                            void* sf_packed, const int32_t* masked_m, int64_t E, int64_t max_m, int64_t I, int64_t K, int64_t expected_m,
                            cudaStream_t st);     // gemm_fp8_mx.cu
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
    uint8_t* a_q; float* a_s;          // quantised local tokens
    __nv_bfloat16* mm1; uint8_t* a2_q; float* a2_s; __nv_bfloat16* mm2;
    uint8_t* sf2;                      // packed UE8M0 scales of the activation between the GEMMs (UE8M0 GEMM path)
    int32_t* identity;                 // [max_tokens*topk] 0,1,2,...
    int32_t* done;                     // [4] block-completion counters of dispatch and combine, the step counter, spare
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

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Publishes `epoch` to flag slot `rank` of every peer once every block of the grid has passed here.
__device__ __forceinline__ void signal_when_grid_done(int32_t* done, const EpPeers& peers, int64_t flags_off, int rank,
                                                      int world, const int32_t* epoch, int32_t* counters_to_clear, int n_clear) {
    __threadfence_system();
    __syncthreads();
    __shared__ int last;
    if (threadIdx.x == 0) last = (atomicAdd(done, 1) == (int)(gridDim.x * gridDim.y) - 1);
    __syncthreads();
    if (!last) return;
    if (counters_to_clear)
        for (int i = threadIdx.x; i < n_clear; i += blockDim.x) counters_to_clear[i] = 0;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < world)
        st_release_sys(reinterpret_cast<int32_t*>(peers.base[threadIdx.x] + flags_off) + rank, *epoch + 1);
    if (threadIdx.x == 0) *done = 0;
}

// One warp per (token, slot) pair of this rank.
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const uint8_t* __restrict__ a_q, const float* __restrict__ a_s, const int32_t* __restrict__ ids,
                   int n_pairs, int topk, int hidden, int e_local, int max_m, int experts_total, EpPeers peers, EpLayout lay,
                   int rank, int world, const int32_t* epoch, int32_t* done, int32_t* status) {
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (i < n_pairs) {
        const int e = ids[i];
        if (e >= 0 && e < experts_total) {
            const int dst = e / e_local, le = e - dst * e_local;
            uint8_t* pb = peers.base[dst];
            int pos = 0;
            if (lane == 0) pos = atomicAdd_system(reinterpret_cast<int32_t*>(pb + lay.counters) + le, 1);
            pos = __shfl_sync(0xffffffffu, pos, 0);
            if (pos < max_m) {
                const int64_t row = (int64_t)le * max_m + pos;
                const int t = i / topk;
                const uint4* src = reinterpret_cast<const uint4*>(a_q + (int64_t)t * hidden);
                uint4* dq = reinterpret_cast<uint4*>(pb + lay.recv_q + row * hidden);
                for (int v = lane; v < (hidden >> 4); v += 32) dq[v] = __ldg(src + v);
                const int g = hidden >> 7;
                float* ds = reinterpret_cast<float*>(pb + lay.recv_s) + row * g;
                // scales twice: fp32 (general GEMM path) and packed UE8M0 words (block-scaled GEMM path):
                // word ((row/128)*g + k)*128 + (row%32)*4 + (row%128)/32, exponent byte repeated
                uint32_t* dp = reinterpret_cast<uint32_t*>(pb + lay.recv_sf) + (size_t)(row >> 7) * g * 128 + (row & 31) * 4 + ((row & 127) >> 5);
                for (int k = lane; k < g; k += 32) {
                    const float sv = __ldg(a_s + (int64_t)t * g + k);
                    ds[k] = sv;
                    dp[(size_t)k * 128] = ((__float_as_uint(sv) >> 23) & 0xffu) * 0x01010101u;
                }
                if (lane == 0) reinterpret_cast<int32_t*>(pb + lay.recv_meta)[row] = (rank << 20) | i;
            } else if (lane == 0) {
                atomicCAS(status, 0, 10);          // an expert received more than max_m rows
                status[3] = e;
            }
        } else if (lane == 0) {
            atomicCAS(status, 0, 11);              // expert id out of range
            status[3] = e;
        }
    }
    signal_when_grid_done(done, peers, lay.flags_dispatch, rank, world, epoch, nullptr, 0);
}

// One block; thread r waits until source r has published `epoch` (or the bound runs out).
// advance != 0 (the step's last wait): once every thread is done, the step counter moves on.
__global__ void ep_wait_kernel(const int32_t* __restrict__ flags, int world, int32_t* epoch_word, int phase, int32_t* status,
                               int advance) {
    const int r = threadIdx.x;
    const int32_t epoch = *epoch_word + 1;
    if (r < world) {
        const long long t0 = clock64();
        while (ld_acquire_sys(flags + r) != epoch) {
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
    __syncthreads();
    if (advance && threadIdx.x == 0) *epoch_word = epoch;
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

__global__ void ep_iota_kernel(int32_t* p, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = i;
}

}  // namespace kbn

extern "C" int kbn_moe_unpermute_combine(const void*, int64_t, const int32_t*, const float*, int64_t, int64_t, int64_t, void*, kbn_stream_t);
extern "C" int kbn_quant_1x128(const void*, int64_t, int64_t, int64_t, void*, int64_t, float*, int64_t, int64_t, float, int, kbn_stream_t);

extern "C" int kbn_ep_create(int rank, int world, int64_t experts_total, int64_t max_m, int64_t hidden, int64_t inter,
                             int64_t max_tokens, int64_t topk, kbn_ep_ctx** out) {
    using namespace kbn;
    KBN_REQUIRE(out, KBN_ERR_ARG, "kbn_ep_create: null out pointer");
    KBN_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, KBN_ERR_ARG, "kbn_ep_create: bad rank/world %d/%d", rank, world);
    KBN_REQUIRE(experts_total > 0 && experts_total % world == 0, KBN_ERR_ARG, "kbn_ep_create: experts (%lld) must divide evenly over %d ranks",
                (long long)experts_total, world);
    KBN_REQUIRE(hidden % 128 == 0 && inter % 128 == 0 && hidden > 0 && inter > 0, KBN_ERR_ARG, "kbn_ep_create: hidden and inter must be multiples of 128");
    KBN_REQUIRE(max_m > 0 && max_tokens > 0 && topk > 0 && max_tokens * topk < (1 << 20), KBN_ERR_ARG, "kbn_ep_create: bad max_m/max_tokens/topk");
    kbn_ep_ctx* c = new (std::nothrow) kbn_ep_ctx();
    KBN_REQUIRE(c, KBN_ERR_CUDA, "kbn_ep_create: out of host memory");
    c->rank = rank; c->world = world;
    c->experts_total = experts_total; c->e_local = experts_total / world; c->max_m = max_m; c->hidden = hidden; c->inter = inter;
    c->max_tokens = max_tokens; c->topk = topk; c->attached = false;
    KBN_CUDA(cudaGetDevice(&c->device));
    c->lay = make_layout(*c);
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->sym), (size_t)c->lay.total));
    KBN_CUDA(cudaMemset(c->sym, 0, (size_t)c->lay.total));
    const int64_t rows = c->e_local * max_m;
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->a_q), (size_t)(max_tokens * hidden)));
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->a_s), (size_t)(max_tokens * (hidden / 128) * 4)));
    c->mm1 = nullptr;      // bf16 GEMM outputs of the fp32-scale path only: allocated by the first call that takes it
    c->mm2 = nullptr;
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->a2_q), (size_t)(rows * inter)));
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->a2_s), (size_t)(rows * (inter / 128) * 4)));
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->sf2), (size_t)kbn_packed_sf_rows_bytes(rows, inter)));
    KBN_CUDA(cudaMemset(c->sf2, 0x7f, (size_t)kbn_packed_sf_rows_bytes(rows, inter)));
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->identity), (size_t)(max_tokens * topk * 4)));
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->done), 16));
    KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->status), 16));
    KBN_CUDA(cudaMemset(c->done, 0, 16));
    c->epoch = c->done + 2;            // words 0 and 1: block-completion counters; word 2: completed steps
    KBN_CUDA(cudaMemset(c->status, 0, 16));
    const int n = (int)(max_tokens * topk);
    ep_iota_kernel<<<(n + 255) / 256, 256>>>(c->identity, n);
    KBN_CHECK_LAUNCH();
    KBN_CUDA(cudaDeviceSynchronize());
    for (int r = 0; r < kMaxRanks; ++r) c->peers.base[r] = nullptr;
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

extern "C" int kbn_ep_moe_forward(kbn_ep_ctx* c, const void* x_bf16, const int32_t* topk_ids, const float* topk_w, int64_t T,
                                  const void* w13, const float* w13_s, const void* w2, const float* w2_s,
                                  const void* w13_sf_packed, const void* w2_sf_packed, void* out_bf16, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(c, KBN_ERR_ARG, "kbn_ep_moe_forward: null context");
    KBN_REQUIRE(c->attached, KBN_ERR_ARG, "kbn_ep_moe_forward: peers not attached (call kbn_ep_attach)");
    KBN_REQUIRE(T >= 0 && T <= c->max_tokens, KBN_ERR_ARG, "kbn_ep_moe_forward: T=%lld exceeds max_tokens=%lld", (long long)T, (long long)c->max_tokens);
    const bool ue8m0 = w13_sf_packed && w2_sf_packed;
    KBN_REQUIRE(w13 && w2 && (ue8m0 || (w13_s && w2_s)), KBN_ERR_ARG, "kbn_ep_moe_forward: null weight pointer");
    KBN_REQUIRE(!ue8m0 || c->max_m % 128 == 0, KBN_ERR_ARG, "kbn_ep_moe_forward: the UE8M0 path needs max_m to be a multiple of 128");
    if (T > 0) KBN_REQUIRE(x_bf16 && topk_ids && topk_w && out_bf16, KBN_ERR_ARG, "kbn_ep_moe_forward: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int32_t* epoch = c->epoch;
    const int H = (int)c->hidden, I = (int)c->inter, G = H / 128;
    uint8_t* mine = c->sym;
    int32_t* counters = reinterpret_cast<int32_t*>(mine + c->lay.counters);
    int rc;
    // 1. quantise the local tokens (row-major scales)
    if (T > 0) {
        rc = kbn_quant_1x128(x_bf16, T, H, H, c->a_q, H, c->a_s, G, 1, 1e-10f, 1, stream);
        if (rc != KBN_OK) return rc;
    }
    // 2. dispatch + signal (at least one block even with no tokens, so that peers are not left waiting)
    const int n_pairs = (int)(T * c->topk);
    const int dblocks = n_pairs > 0 ? (n_pairs + 7) / 8 : 1;
    ep_dispatch_kernel<<<dblocks, 256, 0, st>>>(c->a_q, c->a_s, topk_ids, n_pairs, (int)c->topk, H, (int)c->e_local, (int)c->max_m,
                                                 (int)c->experts_total, c->peers, c->lay, c->rank, c->world, epoch, c->done, c->status);
    KBN_CHECK_LAUNCH();
    // 3. wait for every source's rows
    ep_wait_kernel<<<1, kMaxRanks, 0, st>>>(reinterpret_cast<const int32_t*>(mine + c->lay.flags_dispatch), c->world, epoch, 1, c->status, 0);
    KBN_CHECK_LAUNCH();
    // 4. local experts on the received rows.  Rows per expert to expect if every rank brings as many tokens as this one and
    //    the routing is even: it decides the operand order of the masked GEMMs (few rows: weights as the M operand)
    const int64_t expected_m = std::max<int64_t>(1, (T * c->world * c->topk + c->experts_total - 1) / c->experts_total);
    const float* recv_s = reinterpret_cast<const float*>(mine + c->lay.recv_s);
    if (ue8m0) {
        // GEMM1 with SiLU(gate)*up and the 1x128 quantisation in its epilogue
        rc = mx::gemm1_masked_ue8m0_silu(mine + c->lay.recv_q, mine + c->lay.recv_sf, w13, w13_sf_packed, c->a2_q, c->a2_s, c->sf2, counters,
                                         c->e_local, c->max_m, I, H, expected_m, st);
        if (rc != KBN_OK) return rc;
    } else {
        if (!c->mm1) {
            // Weight scales that are not powers of two (or max_m not a multiple of 128): the GEMMs store bf16 and the
            // activation and the combine are kernels of their own.  Their two scratch buffers are the size of the
            // receive buffers times 2I and H bf16 and are allocated here, once; not inside a stream capture.
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            KBN_CUDA(cudaStreamIsCapturing(st, &cap));
            KBN_REQUIRE(cap == cudaStreamCaptureStatusNone, KBN_ERR_UNSUPPORTED,
                        "kbn_ep_moe_forward: the first call on the fp32-scale path allocates scratch and cannot be captured");
            const int64_t rows = c->e_local * c->max_m;
            KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->mm1), (size_t)(rows * 2 * I * 2)));
            KBN_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->mm2), (size_t)(rows * H * 2)));
        }
        rc = kbn_fp8_grouped_gemm_masked(mine + c->lay.recv_q, recv_s, c->max_m * G, G, 1, w13, w13_s, c->mm1, counters, c->e_local, c->max_m, 2 * I, H, stream);
        if (rc != KBN_OK) return rc;
        rc = silu_mul_quant_masked(c->mm1, c->e_local, c->max_m, I, c->a2_q, c->a2_s, counters, st, nullptr);
        if (rc != KBN_OK) return rc;
    }
    if (ue8m0) {
        // 5. GEMM2 whose epilogue writes every result row straight into its source rank's staging buffer (peer
        //    stores issued tile by tile while the weights of the next tiles stream in) and signals when the grid is done
        CombineEpilogue cb{};
        for (int r = 0; r < c->world; ++r) {
            cb.peer_comb[r] = c->peers.base[r] + c->lay.comb;
            cb.peer_flag[r] = reinterpret_cast<int32_t*>(c->peers.base[r] + c->lay.flags_combine) + c->rank;
        }
        cb.meta = reinterpret_cast<const int32_t*>(mine + c->lay.recv_meta);
        cb.done = c->done + 1;
        cb.counters = counters;
        cb.n_counters = (int32_t)c->e_local;
        cb.world = c->world;
        cb.epoch = epoch;              // the device word
        rc = mx::gemm_masked_ue8m0_combine(c->a2_q, c->sf2, w2, w2_sf_packed, counters, c->e_local, c->max_m, H, I, cb, expected_m, st);
        if (rc != KBN_OK) return rc;
    } else {
        rc = kbn_fp8_grouped_gemm_masked(c->a2_q, c->a2_s, c->max_m * (I / 128), I / 128, 1, w2, w2_s, c->mm2, counters, c->e_local, c->max_m, H, I, stream);
        if (rc != KBN_OK) return rc;
        // 5. results back to their sources + signal; blocks per expert: enough to fill the GPU when a rank owns few
        //    experts with many rows, never more than the rows need
        const unsigned cs_x = (unsigned)std::min<int64_t>((c->max_m + 7) / 8, std::max<int64_t>(8, (4 * (int64_t)sm_count() + c->e_local - 1) / c->e_local));
        ep_combine_send_kernel<<<dim3(cs_x, (unsigned)c->e_local), 256, 0, st>>>(c->mm2, H, (int)c->e_local, (int)c->max_m, c->peers, c->lay, c->rank,
                                                                                c->world, epoch, c->done + 1);
        KBN_CHECK_LAUNCH();
    }
    ep_wait_kernel<<<1, kMaxRanks, 0, st>>>(reinterpret_cast<const int32_t*>(mine + c->lay.flags_combine), c->world, epoch, 2, c->status, 1);
    KBN_CHECK_LAUNCH();
    // 6. weighted sum over the topk slots of each local token, in slot order
    if (T > 0) {
        rc = kbn_moe_unpermute_combine(mine + c->lay.comb, H, c->identity, topk_w, T, c->topk, H, out_bf16, stream);
        if (rc != KBN_OK) return rc;
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

extern "C" int kbn_ep_destroy(kbn_ep_ctx* c) {
    if (!c) return KBN_OK;
    cudaDeviceSynchronize();
    for (int r = 0; r < c->world; ++r)
        if (r != c->rank && c->peers.base[r] && c->peers.base[r] != c->sym) cudaIpcCloseMemHandle(c->peers.base[r]);
    cudaFree(c->sym); cudaFree(c->a_q); cudaFree(c->a_s); cudaFree(c->mm1); cudaFree(c->a2_q); cudaFree(c->a2_s);
    cudaFree(c->mm2); cudaFree(c->sf2); cudaFree(c->identity); cudaFree(c->done); cudaFree(c->status);
    delete c;
    cudaGetLastError();        // a failed release must not surface as the next launch's error
    return KBN_OK;
}
