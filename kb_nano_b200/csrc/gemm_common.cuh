// Tile scheduling and bounded waits shared by the two FP8 GEMM kernels (fp32-scale promotion kernel
// and UE8M0 block-scaled kernel).
#pragma once
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace kbn {

constexpr int kBlockM = 128, kBlockK = 128;
constexpr int kSwizzleGroupM = 8;                        // m-blocks that share B tiles in L2
constexpr long long kWaitLimitCycles = 2000000000ll;     // about a second

enum GemmMode : int { kDense = 0, kContig = 1, kMasked = 2 };

struct GemmParams {
    const float* sa;
    int64_t sa_exp, sa_row, sa_grp;
    const float* sb;
    const __nv_bfloat16* bias;   // dense form only, may be null: bf16 [N], added in fp32 before the result is rounded to bf16
    __nv_bfloat16* C;
    int64_t ldc;
    const int32_t* row_expert;
    const int32_t* masked_m;
    int32_t expected_m;        // masked layout, host side only: rows per expert the caller expects (0: unknown)
    int32_t* status;
    int32_t rows_total;   // rows of the 2-D view of A / C
    int32_t N, K, E, max_m;
    int32_t num_m_blocks, num_n_blocks, num_k_blocks, sb_nb;
    int32_t mode;
    // fused activation epilogue (UE8M0 kernel only): N counts output columns, B holds 2*N rows per expert
    // (gate rows, then up rows); the tile's 128 outputs per row are quantised as one 1x128 group
    uint8_t* act_q;            // e4m3 [rows, N], row stride act_ld
    int64_t act_ld;
    float* act_scale;          // fp32 scales, element strides (act_s_row, act_s_grp)
    int64_t act_s_row, act_s_grp;
    uint32_t* act_packed;      // optional packed UE8M0 copy of the scales
    const uint16_t* act_table; // exactly rounded bf16 SiLU table
};

// Epilogue that returns result rows to the ranks they came from (expert-parallel MoE layer, masked
// layout): row r of the 2-D view goes to row (meta[r] & 0xfffff) of the [pairs, N] bf16 staging buffer of
// rank meta[r] >> 20, written with plain stores through peer mappings.  When every CTA of the grid has
// finished, the last one clears `counters` and publishes `epoch` in this rank's flag slot on every rank.
constexpr int kMaxPeerRanks = 16;
struct CombineEpilogue {
    uint8_t* peer_comb[kMaxPeerRanks];
    int32_t* peer_flag[kMaxPeerRanks];
    const int32_t* meta;
    int32_t* done;
    int32_t* counters;
    const int32_t* epoch;     // device word: the step that is running is *epoch + 1 (see ep_moe.cu)
    int32_t n_counters, world;
};

enum GemmEpilogue : int { kEpiStore = 0, kEpiAct = 1, kEpiCombine = 2 };

// Hooks that tie the two masked grouped GEMMs of the expert-parallel layer to the kernels around them, so that the
// layer needs no kernel of its own between them (all null / zero for every other caller):
//   wait_flags   the kernel does not read the per-expert row counts before every flag [0, wait_world) holds the
//                running step's number (*epoch + 1): the rows of every source rank have arrived.  Bounded; on expiry
//                {20, wait_phase, peer} goes to ep_status and the kernel carries on.
//   sched        tiles are handed out by an atomic counter instead of round-robin, so that CTAs that become resident
//                late (the kernel is launched while its predecessor still runs) take fewer tiles.
//   tile_done    one counter per 128-row block of the masked layout.  done_signal: every epilogue warp adds one after
//                its stores of a tile (GEMM1 + activation).  done_target: the producer loads a tile's rows only once the
//                block's counter has reached it (GEMM2, which reads what GEMM1 wrote while GEMM1 may still run).
struct EpHooks {
    const int32_t* wait_flags;
    const int32_t* epoch;
    int32_t* ep_status;
    int32_t* sched;
    int32_t* tile_done;
    int32_t wait_world, wait_phase;
    int32_t done_signal, done_target;
    unsigned long long* trace;   // debug builds (-DKBN_TRACE) only
};

struct Tile {
    int32_t row0;      // first row in the 2-D view of A and C
    int32_t row_end;   // rows >= row_end are not written
    int32_t n_blk;
    int32_t expert;
    bool compute;      // false: nothing to do for this tile (padding block)
};

// Deterministic tile sequence; every role walks the same one.
struct TileWalk {
    const GemmParams& p;
    int32_t e_cur = 0, blk_base = 0;
    __device__ explicit TileWalk(const GemmParams& pp) : p(pp) {}

    __device__ __forceinline__ int32_t masked_blocks(int32_t e) const {
        int32_t mm = min(max(p.masked_m[e], 0), p.max_m);
        return (mm + kBlockM - 1) / kBlockM;
    }

    __device__ bool get(int64_t t, Tile& tile) {
        if (p.mode == kMasked) {
            int64_t mb = t / p.num_n_blocks;
            tile.n_blk = (int32_t)(t - mb * p.num_n_blocks);
            while (e_cur < p.E) {
                int32_t nb = masked_blocks(e_cur);
                if (mb < (int64_t)blk_base + nb) break;
                blk_base += nb;
                ++e_cur;
            }
            if (e_cur >= p.E) return false;
            tile.expert = e_cur;
            tile.row0 = e_cur * p.max_m + (int32_t)(mb - blk_base) * kBlockM;
            tile.row_end = e_cur * p.max_m + min(max(p.masked_m[e_cur], 0), p.max_m);
            tile.compute = true;
            return true;
        }
        const int64_t total = (int64_t)p.num_m_blocks * p.num_n_blocks;
        if (t >= total) return false;
        const int64_t per_group = (int64_t)kSwizzleGroupM * p.num_n_blocks;
        const int32_t grp = (int32_t)(t / per_group);
        const int32_t first_m = grp * kSwizzleGroupM;
        const int32_t gsz = min(kSwizzleGroupM, p.num_m_blocks - first_m);
        const int32_t within = (int32_t)(t - grp * per_group);
        const int32_t m_blk = first_m + within % gsz;
        tile.n_blk = within / gsz;
        tile.row0 = m_blk * kBlockM;
        tile.row_end = p.rows_total;
        tile.expert = 0;
        tile.compute = true;
        if (p.mode == kContig) {
            int32_t e = p.row_expert[tile.row0];
            tile.expert = e;
            tile.compute = (e >= 0 && e < p.E);
        }
        return true;
    }
};

struct WaitCtx {
    volatile int* abort_flag;   // shared memory
    int32_t* status;            // global
    int code;
};

// Bounded mbarrier wait.  Returns false when the CTA is aborting.
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, const WaitCtx& w) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        if (ptx::mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 0u) {
            if (*w.abort_flag) return false;
            if (clock64() - t0 > kWaitLimitCycles) {
                *w.abort_flag = 1;
                atomicCAS(w.status, 0, w.code | (int)(blockIdx.x << 8));
                return false;
            }
        }
    }
}


// Bounded wait until the counter at `p` (written by other CTAs with release semantics) has reached `target`.
__device__ __forceinline__ bool wait_count(const int32_t* p, int32_t target, const WaitCtx& w) {
    if (ptx::ld_acquire_gpu(p) >= target) return true;
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        if (ptx::ld_acquire_gpu(p) >= target) return true;
        if ((it & 63u) == 0u) {
            if (*w.abort_flag) return false;
            if (clock64() - t0 > kWaitLimitCycles) {
                *w.abort_flag = 1;
                atomicCAS(w.status, 0, w.code | (int)(blockIdx.x << 8));
                return false;
            }
        }
        __nanosleep(32);
    }
}

// Thread `r` of the callers waits until flag r holds the running step's number; see EpHooks.
__device__ __forceinline__ void wait_step_flag(const EpHooks& h, int r) {
    const int32_t want = *h.epoch + 1;
    const long long t0 = clock64();
    while (ptx::ld_acquire_sys(h.wait_flags + r) != want) {
        if (clock64() - t0 > kWaitLimitCycles) {
            if (atomicCAS(h.ep_status, 0, 20) == 0) {
                h.ep_status[1] = h.wait_phase;
                h.ep_status[2] = r;
            }
            break;
        }
        __nanosleep(64);
    }
}

#ifdef KBN_TRACE
// Debug build only: per kernel (4) and CTA (256) four time stamps of the global timer, in a buffer the
// expert-parallel context owns (EpHooks::trace).
__device__ __forceinline__ unsigned long long trace_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define KBN_TRACE_MARK(buf, k, slot) do { if ((buf) != nullptr && threadIdx.x == 0 && blockIdx.x < 256 && blockIdx.y == 0) (buf)[((k) * 256 + blockIdx.x) * 4 + (slot)] = trace_now(); } while (0)
// the same with the step's parity as a fifth index: two consecutive steps are kept
#define KBN_TRACE_MARK2(buf, epoch_ptr, k, slot) do { if ((buf) != nullptr && threadIdx.x == 0 && blockIdx.x < 256 && blockIdx.y == 0) (buf)[4096 * (*(epoch_ptr) & 1) + ((k) * 256 + blockIdx.x) * 4 + (slot)] = trace_now(); } while (0)
#else
#define KBN_TRACE_MARK2(buf, epoch_ptr, k, slot) do { } while (0)
#define KBN_TRACE_MARK(buf, k, slot) do { } while (0)
#endif

// Device status word shared by all GEMM launches of the process (lives in runtime.cu).
int gemm_status_ptr(int32_t** out);

}  // namespace kbn
