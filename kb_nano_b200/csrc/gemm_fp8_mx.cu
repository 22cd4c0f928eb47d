// Block-scaled FP8 GEMM, UE8M0 fast path: when every activation and weight scale is a power of two,
// the scales ride along as UE8M0 bytes in TMEM and the tensor core applies them itself
// (tcgen05.mma.kind::mxf8f6f4.block_scale), so a whole 128x256 (or 128x128) output tile accumulates in
// TMEM over all of K and is read back once.  Same three forms (dense, expert-contiguous, masked) and the
// same tile walk as the fp32-scale kernel.
//
//   warp 0      producer: per K-block one TMA box of A (128 B x 128 rows), one of B (128 B x 256
//               rows), and two plain bulk copies of the packed scale blocks (512 B + 1024 B)
//   warp 1      TMEM allocation; per K-block three tcgen05.cp (scale blocks -> TMEM columns) and
//               four 128x256x32 block-scaled UMMAs
//   warps 2..9  epilogue once per tile: TMEM -> registers -> bf16 -> global
//
// Compared with 128x128 tiles this moves 48 KB instead of 64 KB through L2 per 128x256x128 of work,
// which is what bounds the kernel once the weights stream from HBM.  Packed scale layout (built by
// kbn_pack_sf_*): one 32-bit word per (row, K-block) holding the UE8M0 byte four times, stored per
// 128-row block as [32][4] words so that word (l, i) belongs to row 32*i + l -- the order in which
// tcgen05.cp.32x128b.warpx4 spreads a 512-byte block over TMEM lanes and columns.
#include <cuda.h>

#include <algorithm>

#include "gemm_common.cuh"
#include "silu_exact.cuh"

namespace kbn {
namespace mx {

// Tile width BN is 256 (less L2 traffic per flop; the default) or 128 (twice the tiles: used when a
// dense problem would otherwise leave most SMs without a tile).
constexpr int kStgPitch = 80;                        // bytes per staged row of a 32x32 bf16 chunk (64 B + padding)
constexpr int kEpiScratch = 8 * 32 * kStgPitch;      // 20,480 B: one 32-row staging area per epilogue warp

template <int BN>
struct Cfg {
    static constexpr int kBN = BN;
    static constexpr int kStages = BN == 256 ? 4 : 6;
    static constexpr int kBBytes = BN * kBlockK;
    static constexpr int kStageBytes = kBlockM * kBlockK + kBBytes;
    static constexpr int kSfbBytes = 512 * (BN / 128);
    static constexpr int kSfStage = 512 + kSfbBytes;
    static constexpr int kTxBytes = kStageBytes + kSfStage;
    // 1024: alignment slack; 256: barriers; kEpiScratch: epilogue scratch (absmax exchange or per-warp transposes)
    static constexpr size_t kSmemBytes = (size_t)kStages * (kStageBytes + kSfStage) + 1024 + 256 + kEpiScratch;
};
constexpr int kABytes = kBlockM * kBlockK;          // 16 KB
// Swapped form: a ring slot is 32 KB of weights followed by the token box, and the ring is cut by the live rows of the
// block: 6 slots with a 32-row box, 5 with a 64-row box, 4 with the 128-row box.  The scales (1.5 KB per slot) have
// their own area behind the ring.
constexpr int kSwapWBytes = 256 * kBlockK;
constexpr int kSwapSlotsMax = 6;
constexpr int kSwapMaxExpectedRows = 56;
__host__ __device__ constexpr int swap_class(int live) { return live <= 32 ? 0 : (live <= 64 ? 1 : 2); }
__host__ __device__ constexpr uint32_t swap_slots(int cls) { return 6u - (uint32_t)cls; }
__host__ __device__ constexpr uint32_t swap_slot_bytes(int cls) { return (uint32_t)kSwapWBytes + (32u << cls) * kBlockK; }
constexpr int kSwapRing = 6 * (kSwapWBytes + 32 * kBlockK);      // 221,184 B
constexpr int kSwapSfBytes = 1536;
// ring, scales, alignment slack, barriers, activation exchange: 232,192 B of the 232,448 a CTA can have
constexpr size_t kSwapSmemBytes = (size_t)kSwapRing + kSwapSlotsMax * kSwapSfBytes + 1024 + 256 + 512;
static_assert(swap_slots(1) * swap_slot_bytes(1) <= kSwapRing && swap_slots(2) * swap_slot_bytes(2) <= kSwapRing, "ring");
constexpr int kSfaBytes = 512;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 32 * (2 + kEpiWarps);
// The persistent kernel has one more warp, the tile scheduler of the dynamic schedule (it leaves at once otherwise).
constexpr int kThreadsMain = kThreads + 32;
constexpr int kSchedDepth = 2;                      // tile numbers the scheduler warp may be ahead of their consumers
constexpr int kTmemCols = 512;
constexpr int kColSfa = 256, kColSfb = 260;         // TMEM columns of the scale factors

struct MxExtra {
    const uint8_t* sfa;      // packed [row_blocks][KB][512 B]
    const uint8_t* sfb;      // packed [E][KB][nb_pad][512 B]
    int32_t nb_pad;          // 128-column blocks per expert, rounded up to even
};

// ACT: the tile's B operand is 128 gate rows and the matching 128 up rows of a [2N, K] weight, and the
// epilogue computes y = bf16(bf16(silu(gate)) * up) on the bf16-rounded accumulators and quantises the
// 128 outputs of each row as one 1x128 group (UE8M0 scale, eps 1e-10) -- the same bits as storing the
// bf16 GEMM result and running the stand-alone activation kernel on it, without the round trip.
// EPI == kEpiCombine: instead of storing to C, every result row is written to the rank it came from (see
// CombineEpilogue); 32x32 chunks are transposed through shared memory so that four lanes write 64 contiguous
// bytes of one row, and the grid signals the peers when its last CTA is done.
//
// SWAP (masked form with at most 256 rows per expert, BN = 256): the operands trade places.  The tile's 256 weight
// rows become the M operand of two 128-row MMAs (accumulators at TMEM columns 0 and 128) and the expert's tokens the
// N operand, N = the live rows of the block rounded up to 16; the weights' scale blocks are the A scales, the tokens'
// block the B scales.  A block with 4 live rows then costs an eighth of the tensor work of a 128-row MMA, which is
// what keeps a long run of decode steps under the board's power limit at full clocks.  The accumulator comes out
// transposed: a lane is a weight row = an output column, a TMEM column is a token, so a warp's 32 lanes write 64
// contiguous bytes (bf16) or 32 contiguous bytes (fp8) of one output row.  Without the staging transposes of the
// plain epilogues the shared memory goes to the ring instead: a slot is 32 KB of weights and the token box, and the
// ring holds six of them while blocks have at most 32 live rows (4 KB box), five up to 64 rows and four when a block
// needs the 128-row box; when a tile needs a larger box than any before it in this CTA the producer lets the ring
// run empty and cuts it anew (the cut never goes back to more slots within a launch).
// The epilogue loops over 32-token chunks without unrolling (the common block has one chunk; the code stays small).
// Blocks of at most 64 live rows alternate between two accumulators (AccWalk below).
// Swapped form: which part of TMEM a tile accumulates in.  While a CTA has only seen blocks of at most 64 live rows a
// tile needs 2 x 64 columns and the tiles alternate between columns [0, 128) and [128, 256), so the MMAs of a tile
// start while the epilogue still reads the tile before it; from the first block with more rows on, every tile uses
// all 256 columns (2 x 128) and waits for its predecessor's epilogue.  The MMA issuer and the epilogue warps walk the
// same tiles and keep the same state; bit b of `phases` is the parity of the number of tiles that used accumulator b.
struct AccWalk {
    bool wide = false;
    uint32_t narrow_tiles = 0, phases = 0;
    __device__ __forceinline__ void next(int32_t live, uint32_t& buf, uint32_t& col, uint32_t& sub_stride) {
        if (live > 64) wide = true;
        buf = wide ? 0u : (narrow_tiles++ & 1u);
        col = wide ? 0u : buf * 128u;
        sub_stride = wide ? 128u : 64u;
    }
    __device__ __forceinline__ uint32_t parity(uint32_t buf) const { return (phases >> buf) & 1u; }
    __device__ __forceinline__ void used(uint32_t buf) { phases ^= 1u << buf; }
};

template <int BN, int EPI, bool SWAP>
__global__ void __launch_bounds__(kThreadsMain, 1)
fp8_gemm_mx_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA64,
                   const __grid_constant__ CUtensorMap tmA32, const __grid_constant__ CUtensorMap tmB, const GemmParams p,
                   const MxExtra x, const CombineEpilogue cb, const EpHooks h) {
    static_assert(!SWAP || BN == 256, "the swapped form uses 256 weight rows per tile");
    // expert-parallel layer, dense linear layers: the next kernel of the stream may come in under this one (it waits
    // for this grid's results itself before it reads them)
    if (h.tile_done != nullptr || p.mode == kDense) ptx::launch_dependents();
    KBN_TRACE_MARK2(h.trace, h.epoch, EPI == kEpiCombine ? 2 : 1, 0);
    constexpr bool ACT = EPI == kEpiAct;
    constexpr int kBN = Cfg<BN>::kBN, kStages = Cfg<BN>::kStages, kStageBytes = Cfg<BN>::kStageBytes;
    constexpr int kSfbBytes = Cfg<BN>::kSfbBytes, kSfStage = Cfg<BN>::kSfStage, kTxBytes = Cfg<BN>::kTxBytes;
    constexpr int kHalfCols = BN / 2;                // columns each epilogue warp of a lane quarter drains
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    uint8_t* sf_smem = smem + (size_t)kStages * kStageBytes;
    constexpr int kBars = SWAP ? kSwapSlotsMax : kStages;     // ring barriers of each kind
    uint64_t* bars = reinterpret_cast<uint64_t*>(SWAP ? smem + kSwapRing + kSwapSlotsMax * kSwapSfBytes : sf_smem + (size_t)kStages * kSfStage);
    // bars: full[kBars], empty[kBars], tmem_full, tmem_empty, pair[4] (the two epilogue warps of a lane quarter),
    // tmem_full and tmem_empty of the second accumulator (swapped form), tile-queue full[kSchedDepth] and empty[kSchedDepth]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kBars + 8 + 2 * kSchedDepth);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // Tile queue (dynamic schedule only): the scheduler warp takes tile numbers from the global counter -- and, where a
    // tile's rows come from a kernel that may still be running, waits for them -- and hands the numbers to the producer,
    // the MMA issuer and the epilogue warps through these slots, so that neither the atomic's round trip nor that wait
    // is ever on the path of the thread that keeps the loads in flight.
    volatile int32_t* sched_ids = reinterpret_cast<volatile int32_t*>(tmem_slot + 2);
    static_assert((2 * kBars + 8 + 2 * kSchedDepth) * 8 + 8 + 4 * kSchedDepth <= 256, "barrier block");
    float* xch = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);     // [parity][half][128 rows]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = ptx::smem_u32(bars), bar_empty = ptx::smem_u32(bars + kBars);
    const uint32_t bar_tfull = ptx::smem_u32(bars + 2 * kBars), bar_tempty = ptx::smem_u32(bars + 2 * kBars + 1);
    const uint32_t bar_pair = ptx::smem_u32(bars + 2 * kBars + 2);
    const uint32_t bar_tfull1 = ptx::smem_u32(bars + 2 * kBars + 6), bar_tempty1 = ptx::smem_u32(bars + 2 * kBars + 7);
    const uint32_t bar_sfull = ptx::smem_u32(bars + 2 * kBars + 8), bar_sempty = ptx::smem_u32(bars + 2 * kBars + 8 + kSchedDepth);
    const bool dyn = h.sched != nullptr;
    const uint32_t smem_tiles = ptx::smem_u32(smem), smem_sf = ptx::smem_u32(sf_smem);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kBars; ++s) {
            ptx::mbar_init(bar_full + 8 * s, 1);
            ptx::mbar_init(bar_empty + 8 * s, 1);
        }
        ptx::mbar_init(bar_tfull, 1);
        ptx::mbar_init(bar_tempty, kEpiWarps);
        ptx::mbar_init(bar_tfull1, 1);
        ptx::mbar_init(bar_tempty1, kEpiWarps);
        for (int q = 0; q < 4; ++q) ptx::mbar_init(bar_pair + 8 * q, SWAP ? 4 : 2);   // SWAP: the four quarter warps of a token half
        for (int q = 0; q < kSchedDepth; ++q) {
            ptx::mbar_init(bar_sfull + 8 * q, 1);
            ptx::mbar_init(bar_sempty + 8 * q, 2 + kEpiWarps);       // producer, MMA issuer, epilogue warps
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
        ptx::tmem_relinquish();
    }
    // expert-parallel layer: the row counts and the rows themselves are final once every source rank's flag is up
    if (h.wait_flags != nullptr && warp == 2 && lane < h.wait_world) wait_step_flag(h, lane);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int KB = p.num_k_blocks;
    KBN_TRACE_MARK2(h.trace, h.epoch, EPI == kEpiCombine ? 2 : 1, 1);
    // n-th tile of this CTA for the producer (whole warp), the MMA issuer (one thread) and the epilogue warps (whole
    // warp): round-robin, or the number the scheduler warp has put into the queue
    auto next_tile = [&](uint32_t n, const WaitCtx& w, bool& ok) -> int64_t {
        if (!dyn) return (int64_t)blockIdx.x + (int64_t)n * gridDim.x;
        const uint32_t s = n % kSchedDepth;
        if (!wait_bar(bar_sfull + 8 * s, (n / kSchedDepth) & 1u, w)) { ok = false; return 0; }
        const int32_t t = sched_ids[s];
        if (warp != 1) __syncwarp();
        if (warp == 1 || lane == 0) ptx::mbar_arrive(bar_sempty + 8 * s);
        return t;
    };

    if (warp == 0) {
        // ---------------- producer ----------------
        // The whole warp walks the tiles (so that it can look at a block's 128 row ids with one load per
        // lane); lane 0 alone waits on the ring and issues the copies.
        if (lane == 0) {
            ptx::prefetch_tensormap(&tmA);
            ptx::prefetch_tensormap(&tmA64);
            ptx::prefetch_tensormap(&tmA32);
            ptx::prefetch_tensormap(&tmB);
        }
        WaitCtx w{abort_flag, p.status, 4};
        TileWalk walk(p);
        Tile tile;
        uint32_t it = 0;
        // dense form: launched while the kernel before it may still be running (programmatic stream serialisation); its
        // results (the activations this kernel reads, the buffer it writes) are final once this returns
        if (p.mode == kDense) ptx::grid_dependency_wait();
        uint32_t slot = 0, fills = 0;     // SWAP: next ring slot; bit s = parity of the number of fills of slot s
        int cur_cls = -1;                 // SWAP: how the ring is cut at the moment
        bool ok = true;
        for (uint32_t n_tile = 0; ok; ++n_tile) {
            const int64_t t = next_tile(n_tile, w, ok);
            if (!ok || !walk.get(t, tile)) break;
            if (!tile.compute) continue;
            // Rows of the block that hold data: a block with few of them (decode batches, the last block
            // of an expert) fetches a 32- or 64-row box of A instead of 128 rows.  The rest of the stage
            // keeps whatever an earlier tile left there; those accumulator rows are never used.
            int32_t live = min(tile.row_end - tile.row0, kBlockM);
            if (p.mode == kContig) {
                int32_t last = -1;                  // last row of the block with a valid expert id
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int32_t r = 4 * lane + j;
                    if (r < live && p.row_expert[tile.row0 + r] >= 0) last = r;
                }
                live = __reduce_max_sync(0xffffffffu, last) + 1;
            }
            if (lane == 0) {
                // ACT: n_blk counts 128 output columns; gate rows of the expert come first, up rows N later
                const int32_t b_row = ACT ? tile.expert * 2 * p.N + tile.n_blk * 128 : tile.expert * p.N + tile.n_blk * kBN;
                const uint8_t* sfa = x.sfa + (int64_t)(tile.row0 / kBlockM) * KB * kSfaBytes;
                const uint8_t* sfb = x.sfb + (((int64_t)tile.expert * KB) * x.nb_pad + (ACT ? 1 : BN / 128) * tile.n_blk) * (int64_t)kSfaBytes;
                const CUtensorMap* tma = live <= 32 ? &tmA32 : (live <= 64 ? &tmA64 : &tmA);
                const uint32_t tx = (uint32_t)(kTxBytes - kABytes) + (live <= 32 ? 32u : (live <= 64 ? 64u : 128u)) * (uint32_t)kBlockK;
                // the cut only ever grows coarser within a launch: going back and forth between tiles would let the ring
                // run empty every time
                // the block's rows may have been written a moment ago by the kernel before this one (the scheduler warp
                // has seen them counted): order those generic-proxy writes before this thread's bulk loads
                if (h.done_target > 0) ptx::fence_proxy_async_global();
                const int cls = max(swap_class(live), cur_cls);
                if (SWAP && cls != cur_cls) {
                    // the ring is cut differently from here on: wait until every slot in use has been consumed
                    for (int s = 0; s < kBars && ok; ++s) ok = wait_bar(bar_empty + 8 * s, ((fills >> s) & 1u) ^ 1u, w);
                    cur_cls = cls;
                    slot = 0;
                }
                for (int kb = 0; ok && kb < KB; ++kb, ++it) {
                    uint32_t s, w_dst, a_dst, sdst;      // ring slot; where the weight tile, the token box and the scales go
                    if (SWAP) {
                        s = slot;
                        slot = slot + 1 == swap_slots(cls) ? 0u : slot + 1;
                        if (!wait_bar(bar_empty + 8 * s, ((fills >> s) & 1u) ^ 1u, w)) { ok = false; break; }
                        fills ^= 1u << s;
                        w_dst = smem_tiles + s * swap_slot_bytes(cls);
                        a_dst = w_dst + kSwapWBytes;
                        sdst = smem_tiles + kSwapRing + s * kSwapSfBytes;
                    } else {
                        s = it % kStages;
                        if (!wait_bar(bar_empty + 8 * s, ((it / kStages) & 1u) ^ 1u, w)) { ok = false; break; }
                        a_dst = smem_tiles + s * kStageBytes;
                        w_dst = a_dst + kABytes;
                        sdst = smem_sf + s * kSfStage;
                    }
                    const uint32_t bar = bar_full + 8 * s;
                    ptx::mbar_arrive_expect_tx(bar, tx);
                    ptx::tma_load_2d(a_dst, tma, kb * kBlockK, tile.row0, bar);
                    ptx::bulk_load(sdst, sfa + (int64_t)kb * kSfaBytes, kSfaBytes, bar);
                    if (ACT) {
                        // tmB's box is 128 rows here: gate rows fill the first half of the B tile, up rows the second
                        ptx::tma_load_2d(w_dst, &tmB, kb * kBlockK, b_row, bar);
                        ptx::tma_load_2d(w_dst + 128 * kBlockK, &tmB, kb * kBlockK, b_row + p.N, bar);
                        const uint8_t* sg = sfb + (int64_t)kb * x.nb_pad * kSfaBytes;
                        ptx::bulk_load(sdst + kSfaBytes, sg, kSfaBytes, bar);
                        ptx::bulk_load(sdst + 2 * kSfaBytes, sg + (int64_t)(p.N / 128) * kSfaBytes, kSfaBytes, bar);
                    } else {
                        ptx::tma_load_2d(w_dst, &tmB, kb * kBlockK, b_row, bar);
                        ptx::bulk_load(sdst + kSfaBytes, sfb + (int64_t)kb * x.nb_pad * kSfaBytes, kSfbBytes, bar);
                    }
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        if (!ok && lane == 0) {
            const long long t0 = clock64();
            while (clock64() - t0 < 400000ll) __nanosleep(1000);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            WaitCtx w{abort_flag, p.status, 5};
            TileWalk walk(p);
            Tile tile;
            uint32_t it = 0, tile_it = 0;
            uint32_t slot = 0, drains = 0;    // SWAP: next ring slot; bit s = parity of the number of times slot s was consumed
            int cur_cls = -1;
            AccWalk acc;                      // SWAP: which accumulator the tile uses
            constexpr uint32_t idesc = ptx::umma_idesc_mx_e4m3(kBlockM, kBN, 0, 0);
            bool ok = true;
            for (uint32_t n_tile = 0; ok; ++n_tile) {
                const int64_t t = next_tile(n_tile, w, ok);
                if (!ok || !walk.get(t, tile)) break;
                if (!tile.compute) continue;
                // the tile's accumulator must have been drained by the epilogue of the tile that used it last
                const int32_t live_rows = min(tile.row_end - tile.row0, kBlockM);
                uint32_t acc_col = 0, acc_sub = 128, acc_buf = 0;
                if (SWAP) {
                    const bool was_wide = acc.wide;
                    acc.next(live_rows, acc_buf, acc_col, acc_sub);
                    if (acc.wide && !was_wide && !wait_bar(bar_tempty1, acc.parity(1) ^ 1u, w)) { ok = false; break; }   // both halves of TMEM from here on
                    if (!wait_bar(acc_buf ? bar_tempty1 : bar_tempty, acc.parity(acc_buf) ^ 1u, w)) { ok = false; break; }
                } else if (!wait_bar(bar_tempty, (tile_it & 1u) ^ 1u, w)) { ok = false; break; }
                ptx::tc_fence_after();
                // SWAP: N of the instruction = live rows of the block, rounded up to 16
                const uint32_t swap_idesc =
                    ptx::umma_idesc_mx_e4m3(kBlockM, (uint32_t)max(16, (min(tile.row_end - tile.row0, kBlockM) + 15) & ~15), 0, 0);
                const int cls = max(swap_class(min(tile.row_end - tile.row0, kBlockM)), cur_cls);
                if (SWAP && cls != cur_cls) {     // the producer cuts the ring anew and starts at its first slot
                    cur_cls = cls;
                    slot = 0;
                }
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    uint32_t s, ph, a_addr, w_addr, sf_addr;   // ring slot, its phase; token box, weight tile, scales
                    if (SWAP) {
                        s = slot;
                        slot = slot + 1 == swap_slots(cls) ? 0u : slot + 1;
                        ph = (drains >> s) & 1u;
                        drains ^= 1u << s;
                        w_addr = smem_tiles + s * swap_slot_bytes(cls);
                        a_addr = w_addr + kSwapWBytes;
                        sf_addr = smem_tiles + kSwapRing + s * kSwapSfBytes;
                    } else {
                        s = it % kStages;
                        ph = (it / kStages) & 1u;
                        a_addr = smem_tiles + s * kStageBytes;
                        w_addr = a_addr + kABytes;
                        sf_addr = smem_sf + s * kSfStage;
                    }
                    if (!wait_bar(bar_full + 8 * s, ph, w)) { ok = false; break; }
                    ptx::tc_fence_after();
                    ptx::tmem_cp_32x128b_warpx4(tmem_base + kColSfa, ptx::umma_desc_sf(sf_addr));
                    ptx::tmem_cp_32x128b_warpx4(tmem_base + kColSfb, ptx::umma_desc_sf(sf_addr + kSfaBytes));
                    if (BN == 256)
                        ptx::tmem_cp_32x128b_warpx4(tmem_base + kColSfb + 4, ptx::umma_desc_sf(sf_addr + 2 * kSfaBytes));
                    const uint64_t a_desc = ptx::umma_desc_k_sw128(a_addr);
                    const uint64_t b_desc = ptx::umma_desc_k_sw128(w_addr);
                    if (SWAP) {
                        // weights (two 128-row blocks, one accumulator each) x tokens^T: the weights' scale blocks are the A
                        // scales, the tokens' block the B scale; the two accumulators take turns (measured: no faster than one
                        // after the other, kept because consecutive instructions then never depend on each other)
                        const uint64_t w_desc = b_desc;
                        constexpr uint64_t kSubDesc = (128 * kBlockK) >> 4;          // second 128 weight rows, in descriptor units
#pragma unroll
                        for (int k = 0; k < kBlockK / 32; ++k)
#pragma unroll
                            for (int sub = 0; sub < 2; ++sub)
                                ptx::mma_mxf8f6f4_block_scale(tmem_base + acc_col + sub * acc_sub, w_desc + sub * kSubDesc + 2 * k, a_desc + 2 * k, swap_idesc,
                                                              tmem_base + kColSfb + 4 * sub, tmem_base + kColSfa, (kb > 0 || k > 0) ? 1u : 0u);
                    } else {
#pragma unroll
                        for (int k = 0; k < kBlockK / 32; ++k)
                            ptx::mma_mxf8f6f4_block_scale(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, tmem_base + kColSfa,
                                                          tmem_base + kColSfb, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    ptx::mma_commit(bar_empty + 8 * s);
                }
                if (!ok) break;
                ptx::mma_commit(acc_buf ? bar_tfull1 : bar_tfull);
                if (SWAP) acc.used(acc_buf);
                ++tile_it;
            }
        }
    } else if (warp == 2 + kEpiWarps) {
        // ---------------- tile scheduler (dynamic schedule only) ----------------
        if (dyn && lane == 0) {
            WaitCtx w{abort_flag, p.status, 7};
            TileWalk walk(p);
            Tile tile;
            for (uint32_t n = 0;; ++n) {
                const uint32_t s = n % kSchedDepth;
                if (!wait_bar(bar_sempty + 8 * s, ((n / kSchedDepth) & 1u) ^ 1u, w)) break;
                const int32_t t = atomicAdd(h.sched, 1);
                const bool more = walk.get(t, tile);
                // GEMM2 of the expert-parallel layer: the tile's rows are complete once every epilogue warp of every
                // GEMM1 tile of the block has counted itself
                if (more && tile.compute && h.done_target > 0 && !wait_count(h.tile_done + (tile.row0 >> 7), h.done_target, w)) break;
                sched_ids[s] = t;
                ptx::mbar_arrive(bar_sfull + 8 * s);
                if (!more) break;          // the consumers see the same number and stop as well
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;            // which half of the tile's columns this warp drains
        const int r_in_tile = quarter * 32 + lane;
        WaitCtx w{abort_flag, p.status, 6};
        TileWalk walk(p);
        Tile tile;
        uint32_t tile_it = 0, act_it = 0;
        AccWalk acc;                                  // SWAP: which accumulator the tile uses (same walk as the MMA issuer's)
        bool ok = true;
        // GEMM1 of the expert-parallel layer: this warp's stores of a tile are done, count it for the block's rows
        auto tile_stored = [&](const Tile& tl) {
            if (h.done_signal) {
                ptx::fence_proxy_async_global();
                __syncwarp();
                if (lane == 0) ptx::red_release_gpu_add(h.tile_done + (tl.row0 >> 7), 1);
            }
        };
        for (uint32_t n_tile = 0; ok; ++n_tile) {
            const int64_t t = next_tile(n_tile, w, ok);
            if (!ok || !walk.get(t, tile)) break;
            if (!tile.compute) continue;
            const int32_t row = tile.row0 + r_in_tile;
            bool row_ok = row < tile.row_end;
            if (p.mode == kContig && row_ok) row_ok = p.row_expert[row] >= 0;
            uint32_t acc_col = 0, acc_sub = 128, acc_buf = 0;
            if (SWAP) {
                acc.next(min(tile.row_end - tile.row0, kBlockM), acc_buf, acc_col, acc_sub);
                if (!wait_bar(acc_buf ? bar_tfull1 : bar_tfull, acc.parity(acc_buf), w)) { ok = false; break; }
                acc.used(acc_buf);
            } else if (!wait_bar(bar_tfull, tile_it & 1u, w)) { ok = false; break; }
            ptx::tc_fence_after();
            if (SWAP) {
                // Transposed accumulators: lane = weight row (output column), TMEM column = token of the block.
                const int32_t live = min(tile.row_end - tile.row0, kBlockM);
                const int32_t nchunks = (live + 31) >> 5;                 // 32-token chunks that hold data
                const uint32_t tlane = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc_col;
                const uint32_t bar_acc_empty = acc_buf ? bar_tempty1 : bar_tempty;
                if (!ACT) {
                    // warps 2..5 drain the first 128 weight rows, warps 6..9 the second 128, in 32-token chunks
                    const int sub = half;
                    const int32_t n = tile.n_blk * kBN + sub * 128 + quarter * 32 + lane;        // output column
                    const bool n_ok = n < p.N;
                    // combine: where a chunk's 32 tokens go is read with one load per lane and handed round by shuffles (a load
                    // per token in the store loop could not be moved above the stores before it)
                    auto chunk_meta = [&](int c) -> int32_t {
                        return (EPI == kEpiCombine && 32 * c + lane < live) ? cb.meta[tile.row0 + 32 * c + lane] : 0;
                    };
                    auto store_chunk = [&](int c, const uint32_t (&r)[32], int32_t my_meta) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int32_t t = 32 * c + j;
                            if (t >= live) break;
                            const __nv_bfloat16 v = __float2bfloat16_rn(__uint_as_float(r[j]));
                            if (EPI == kEpiCombine) {
                                const int32_t meta = __shfl_sync(0xffffffffu, my_meta, j);
                                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(cb.peer_comb[meta >> 20]) + (int64_t)(meta & 0xfffff) * p.N;
                                if (n_ok) dst[n] = v;                                        // 64 contiguous bytes per warp
                            } else if (n_ok) {
                                p.C[(int64_t)(tile.row0 + t) * p.ldc + n] = v;
                            }
                        }
                    };
                    if (nchunks <= 2) {
                        // the common block: one chunk at a time in a loop that is not unrolled (small code; the producer's and the
                        // MMA issuer's loops stay in the instruction cache), the accumulator handed back after the last read
#pragma unroll 1
                        for (int c = 0; c < nchunks; ++c) {
                            uint32_t r[32];
                            ptx::tmem_ld_32x32(tlane + sub * acc_sub + 32 * c, r);
                            const int32_t my_meta = chunk_meta(c);
                            ptx::tmem_ld_wait(r);
                            if (c == nchunks - 1) {
                                ptx::tc_fence_before();
                                __syncwarp();
                                if (lane == 0) ptx::mbar_arrive(bar_acc_empty);
                            }
                            store_chunk(c, r, my_meta);
                        }
                    } else {
                        // 65..128 live rows: everything into registers first, so that the accumulator goes back before the stores
                        uint32_t r[4][32];
                        int32_t mm[4];
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            if (c < nchunks) {
                                ptx::tmem_ld_32x32(tlane + sub * acc_sub + 32 * c, r[c]);
                                mm[c] = chunk_meta(c);
                            }
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            if (c < nchunks) ptx::tmem_ld_wait(r[c]);
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(bar_acc_empty);
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            if (c < nchunks) store_chunk(c, r[c], mm[c]);
                    }
                } else {
                    // ACT: gate accumulators at columns 0.., up at 128.. .  The two warps of a lane quarter split every 32-token
                    // chunk of the block: warp `half` takes tokens 16 * half .. + 15 of chunk c, for its 32 weight rows, from both
                    // accumulators (one warp per scheduler partition working alone runs at the latency of its own dependent
                    // instructions, so the work is spread over all eight warps and kept short).
                    const int32_t my_chunks = (live - 16 * half + 31) >> 5;                      // chunks with tokens for this warp
                    if (my_chunks <= 0) {
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(bar_acc_empty);
                    }
                    uint32_t* xq = reinterpret_cast<uint32_t*>(xch);                              // [parity][half][quarter][8 words]
                    // One chunk at a time, as a loop that is not unrolled: the code of a chunk is fetched once and stays in
                    // the instruction cache next to the producer's and the MMA issuer's loops.  The accumulator goes back to
                    // the MMA warp when the last chunk has been read.
#pragma unroll 1
                    for (int c = 0; c < my_chunks; ++c) {
                        uint32_t g[16], u[16];
                        ptx::tmem_ld_32x16(tlane + 32 * c + 16 * half, g);
                        ptx::tmem_ld_32x16(tlane + acc_sub + 32 * c + 16 * half, u);
                        ptx::tmem_ld_wait(g);
                        ptx::tmem_ld_wait(u);
                        if (c == my_chunks - 1) {
                            ptx::tc_fence_before();
                            __syncwarp();
                            if (lane == 0) ptx::mbar_arrive(bar_acc_empty);
                        }
                        const int32_t t0 = 32 * c + 16 * half;                                   // first token of the warp's 16
                        // y for 16 tokens of this weight row, two tokens per word
                        uint32_t y[8];
#pragma unroll
                        for (int j = 0; j < 16; j += 8) {
                            uint4 g4, u4;
                            g4.x = pack_bf16x2(__uint_as_float(g[j + 0]), __uint_as_float(g[j + 1]));
                            g4.y = pack_bf16x2(__uint_as_float(g[j + 2]), __uint_as_float(g[j + 3]));
                            g4.z = pack_bf16x2(__uint_as_float(g[j + 4]), __uint_as_float(g[j + 5]));
                            g4.w = pack_bf16x2(__uint_as_float(g[j + 6]), __uint_as_float(g[j + 7]));
                            u4.x = pack_bf16x2(__uint_as_float(u[j + 0]), __uint_as_float(u[j + 1]));
                            u4.y = pack_bf16x2(__uint_as_float(u[j + 2]), __uint_as_float(u[j + 3]));
                            u4.z = pack_bf16x2(__uint_as_float(u[j + 4]), __uint_as_float(u[j + 5]));
                            u4.w = pack_bf16x2(__uint_as_float(u[j + 6]), __uint_as_float(u[j + 7]));
                            uint32_t y4[4];
                            silu_mul_8(g4, u4, p.act_table, y4);
#pragma unroll
                            for (int q4 = 0; q4 < 4; ++q4) y[j / 2 + q4] = y4[q4];
                        }
                        // Per-token absmax over the 128 weight rows of the group.  Within the warp a halving exchange: each
                        // round a lane keeps half of its words and gets the partner's maxima for them (4 + 2 + 1 shuffles), two
                        // plain rounds finish; lane l then holds word 4*bit4(l) + 2*bit3(l) + bit2(l), reduced over all 32 lanes.
                        uint32_t m4[4], m2[2], m1;
                        {
                            const bool hi = (lane & 16) != 0;
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const uint32_t send = hi ? y[i] : y[i + 4], keep = hi ? y[i + 4] : y[i];
                                m4[i] = absmax_bf16x2(keep, __shfl_xor_sync(0xffffffffu, send, 16));
                            }
                        }
                        {
                            const bool hi = (lane & 8) != 0;
#pragma unroll
                            for (int i = 0; i < 2; ++i) {
                                const uint32_t send = hi ? m4[i] : m4[i + 2], keep = hi ? m4[i + 2] : m4[i];
                                m2[i] = absmax_bf16x2(keep, __shfl_xor_sync(0xffffffffu, send, 8));
                            }
                        }
                        {
                            const bool hi = (lane & 4) != 0;
                            const uint32_t send = hi ? m2[0] : m2[1], keep = hi ? m2[1] : m2[0];
                            m1 = absmax_bf16x2(keep, __shfl_xor_sync(0xffffffffu, send, 4));
                        }
                        m1 = absmax_bf16x2(m1, __shfl_xor_sync(0xffffffffu, m1, 2));
                        m1 = absmax_bf16x2(m1, __shfl_xor_sync(0xffffffffu, m1, 1));
                        // the four quarter warps of this half meet in shared memory
                        const uint32_t par = act_it & 1u;
                        ++act_it;
                        uint32_t* grp = xq + (par * 2u + (uint32_t)half) * 32u;
                        if ((lane & 3) == 0) grp[quarter * 8 + (lane >> 2)] = abs_bf16x2(m1);
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(bar_pair + 8 * half);
                        if (!wait_bar(bar_pair + 8 * half, par, w)) { ok = false; break; }
                        // lane t < 16: scale of token t0 + t
                        const int tl = lane & 15;
                        uint32_t wmax = 0;
#pragma unroll
                        for (int qq = 0; qq < 4; ++qq) wmax = max_bf16x2(wmax, grp[qq * 8 + (tl >> 1)]);
                        const float amax = fmaxf((tl & 1) ? bf16_hi(wmax) : bf16_lo(wmax), 1e-10f);
                        const uint32_t f = ue8m0_scale_field(amax);
                        const float inv = __uint_as_float((254u - f) << 23);                    // lanes t and t + 16: token t0 + t
                        const int32_t trow = tile.row0 + t0 + lane;
                        if (quarter == 0 && lane < 16 && t0 + lane < live) {
                            p.act_scale[(int64_t)trow * p.act_s_row + (int64_t)tile.n_blk * p.act_s_grp] = __uint_as_float(f << 23);
                            if (p.act_packed != nullptr)
                                p.act_packed[((size_t)(trow >> 7) * p.num_n_blocks + tile.n_blk) * 128u + (trow & 31) * 4 + ((trow & 127) >> 5)] =
                                    f * 0x01010101u;
                        }
                        // this lane's weight row for every token: one fp8 byte each, 32 contiguous bytes per warp and token
                        uint8_t* qcol = p.act_q + tile.n_blk * 128 + quarter * 32 + lane;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int32_t t = t0 + 2 * i;
                            if (t >= live) break;
                            const float i0 = __shfl_sync(0xffffffffu, inv, 2 * i), i1 = __shfl_sync(0xffffffffu, inv, 2 * i + 1);
                            const uint32_t b2 = pack_e4m3x2(__fmul_rn(bf16_lo(y[i]), i0), __fmul_rn(bf16_hi(y[i]), i1));
                            qcol[(int64_t)(tile.row0 + t) * p.act_ld] = (uint8_t)(b2 & 0xffu);
                            if (t + 1 < live) qcol[(int64_t)(tile.row0 + t + 1) * p.act_ld] = (uint8_t)(b2 >> 8);
                        }
                        __syncwarp();
                    }
                    if (!ok) break;
                }
                tile_stored(tile);
                ++tile_it;
                continue;
            }
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + half * kHalfCols;
            const int32_t n0 = tile.n_blk * kBN + half * kHalfCols;
            __nv_bfloat16* crow = p.C + (int64_t)row * p.ldc + n0;
            const bool vec_ok = (reinterpret_cast<uintptr_t>(crow) & 15u) == 0;
            // Drain first, convert later: all of this warp's columns go to registers with back-to-back TMEM
            // loads, the accumulator is handed back to the MMA warp at once, and the bf16 conversion and the
            // global stores overlap the next tile's MMAs.
            constexpr int kChunks = kHalfCols / 32;
            uint32_t r[kChunks][32];
            if (ACT) {
                // gate columns [64*half, +64) into r[0..1], the matching up columns (128 further) into r[2..3]
                const uint32_t tq = tmem_base + ((uint32_t)(quarter * 32) << 16) + half * 64;
#pragma unroll
                for (int c = 0; c < kChunks; ++c) ptx::tmem_ld_32x32(tq + (c >> 1) * 128 + (c & 1) * 32, r[c]);
            } else {
#pragma unroll
                for (int c = 0; c < kChunks; ++c) ptx::tmem_ld_32x32(taddr + 32 * c, r[c]);
            }
#pragma unroll
            for (int c = 0; c < kChunks; ++c) ptx::tmem_ld_wait(r[c]);
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar_tempty);
            if (ACT) {
                // y = bf16(bf16(silu(bf16(gate))) * bf16(up)) for this thread's 64 outputs, packed two per word
                uint32_t y[32];
#pragma unroll
                for (int c = 0; c < 2; ++c)
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint4 g, u;
                        g.x = pack_bf16x2(__uint_as_float(r[c][j + 0]), __uint_as_float(r[c][j + 1]));
                        g.y = pack_bf16x2(__uint_as_float(r[c][j + 2]), __uint_as_float(r[c][j + 3]));
                        g.z = pack_bf16x2(__uint_as_float(r[c][j + 4]), __uint_as_float(r[c][j + 5]));
                        g.w = pack_bf16x2(__uint_as_float(r[c][j + 6]), __uint_as_float(r[c][j + 7]));
                        u.x = pack_bf16x2(__uint_as_float(r[2 + c][j + 0]), __uint_as_float(r[2 + c][j + 1]));
                        u.y = pack_bf16x2(__uint_as_float(r[2 + c][j + 2]), __uint_as_float(r[2 + c][j + 3]));
                        u.z = pack_bf16x2(__uint_as_float(r[2 + c][j + 4]), __uint_as_float(r[2 + c][j + 5]));
                        u.w = pack_bf16x2(__uint_as_float(r[2 + c][j + 6]), __uint_as_float(r[2 + c][j + 7]));
                        uint32_t y4[4];
                        silu_mul_8(g, u, p.act_table, y4);
#pragma unroll
                        for (int q = 0; q < 4; ++q) y[(c * 32 + j) / 2 + q] = y4[q];
                    }
                uint32_t m2 = y[0];
#pragma unroll
                for (int i = 1; i < 32; ++i) m2 = absmax_bf16x2(m2, y[i]);
                m2 = abs_bf16x2(m2);
                float amax = fmaxf(bf16_lo(m2), bf16_hi(m2));
                // the other half of the row's 128 outputs sits in the partner warp of this lane quarter
                const uint32_t par = act_it & 1u;
                ++act_it;
                xch[(par * 2u + (uint32_t)half) * 128u + (uint32_t)r_in_tile] = amax;
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar_pair + 8 * quarter);
                if (!wait_bar(bar_pair + 8 * quarter, par, w)) { ok = false; break; }
                amax = fmaxf(fmaxf(amax, xch[(par * 2u + (uint32_t)(half ^ 1)) * 128u + (uint32_t)r_in_tile]), 1e-10f);
                const uint32_t f = ue8m0_scale_field(amax);
                const float inv = __uint_as_float((254u - f) << 23);
                if (row_ok) {
                    uint8_t* qrow = p.act_q + (int64_t)row * p.act_ld + tile.n_blk * 128 + half * 64;
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint32_t o[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint32_t w0 = y[i + 2 * q], w1 = y[i + 2 * q + 1];
                            o[q] = pack_e4m3x2(__fmul_rn(bf16_lo(w0), inv), __fmul_rn(bf16_hi(w0), inv)) |
                                   (pack_e4m3x2(__fmul_rn(bf16_lo(w1), inv), __fmul_rn(bf16_hi(w1), inv)) << 16);
                        }
                        *reinterpret_cast<uint4*>(qrow + 2 * i) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                    if (half == 0) {
                        p.act_scale[(int64_t)row * p.act_s_row + (int64_t)tile.n_blk * p.act_s_grp] = __uint_as_float(f << 23);
                        if (p.act_packed != nullptr)
                            p.act_packed[((size_t)(row >> 7) * p.num_n_blocks + tile.n_blk) * 128u + (row & 31) * 4 + ((row & 127) >> 5)] =
                                f * 0x01010101u;
                    }
                }
            } else if (EPI == kEpiCombine) {
                uint8_t* dst_row = nullptr;
                if (row_ok) {
                    const int32_t meta = cb.meta[row];
                    dst_row = cb.peer_comb[meta >> 20] + (int64_t)(meta & 0xfffff) * p.N * 2;
                }
                uint8_t* stg = reinterpret_cast<uint8_t*>(xch) + (warp - 2) * (32 * kStgPitch);
#pragma unroll
                for (int c = 0; c < kChunks; ++c) {
                    const int32_t col0 = n0 + 32 * c;
                    if (col0 >= p.N) break;                            // warp-uniform (N is a multiple of 32 here)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        uint4 v;
                        v.x = pack_bf16x2(__uint_as_float(r[c][8 * k + 0]), __uint_as_float(r[c][8 * k + 1]));
                        v.y = pack_bf16x2(__uint_as_float(r[c][8 * k + 2]), __uint_as_float(r[c][8 * k + 3]));
                        v.z = pack_bf16x2(__uint_as_float(r[c][8 * k + 4]), __uint_as_float(r[c][8 * k + 5]));
                        v.w = pack_bf16x2(__uint_as_float(r[c][8 * k + 6]), __uint_as_float(r[c][8 * k + 7]));
                        *reinterpret_cast<uint4*>(stg + lane * kStgPitch + 16 * k) = v;
                    }
                    __syncwarp();
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int rr = (lane >> 2) + 8 * k, seg = lane & 3;
                        const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * kStgPitch + 16 * seg);
                        const uint64_t d = __shfl_sync(0xffffffffu, reinterpret_cast<uint64_t>(dst_row), rr);
                        if (d != 0) *reinterpret_cast<uint4*>(d + (uint64_t)(col0 + 8 * seg) * 2u) = v;
                    }
                    __syncwarp();
                }
            } else if (row_ok) {
#pragma unroll
                for (int c = 0; c < kChunks; ++c) {
                    if (p.bias != nullptr) {
                        // dense linear layer with a bias: added to the fp32 accumulators, one rounding to bf16 afterwards
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (n0 + 32 * c + j < p.N)
                                r[c][j] = __float_as_uint(__uint_as_float(r[c][j]) + __bfloat162float(p.bias[n0 + 32 * c + j]));
                    }
                    if (n0 + 32 * c + 32 <= p.N && vec_ok) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint4 v;
                            v.x = pack_bf16x2(__uint_as_float(r[c][j + 0]), __uint_as_float(r[c][j + 1]));
                            v.y = pack_bf16x2(__uint_as_float(r[c][j + 2]), __uint_as_float(r[c][j + 3]));
                            v.z = pack_bf16x2(__uint_as_float(r[c][j + 4]), __uint_as_float(r[c][j + 5]));
                            v.w = pack_bf16x2(__uint_as_float(r[c][j + 6]), __uint_as_float(r[c][j + 7]));
                            *reinterpret_cast<uint4*>(crow + 32 * c + j) = v;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (n0 + 32 * c + j < p.N) crow[32 * c + j] = __float2bfloat16_rn(__uint_as_float(r[c][j]));
                    }
                }
            }
            tile_stored(tile);
            ++tile_it;
        }
    }

    // Started while the kernel before it in the stream was still running: this grid must not be seen as complete before
    // that one is, because the kernel after both of them reuses the counters of both.
    ptx::tc_fence_before();
    __syncthreads();
    KBN_TRACE_MARK2(h.trace, h.epoch, EPI == kEpiCombine ? 2 : 1, 2);
    if (h.tile_done != nullptr) {
        ptx::grid_dependency_wait();
        __syncthreads();
    }
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
    if (EPI == kEpiCombine) {
        // Last CTA of the grid: every CTA has read the row counts and sent its rows.  One system-wide fence per CTA,
        // by the thread that counts the CTA: the barrier above has ordered every other thread's peer stores before it
        // (a fence by each of the CTA's threads costs ten microseconds at the end of every launch).
        __shared__ int last;
        if (threadIdx.x == 0) {
            __threadfence_system();
            last = (atomicAdd(cb.done, 1) == (int)gridDim.x - 1);
        }
        __syncthreads();
        if (!last) return;
        for (int i = threadIdx.x; i < cb.n_counters; i += blockDim.x) cb.counters[i] = 0;
        __syncthreads();
        if (threadIdx.x == 0) {
            // one fence: acquire side of the count just read, release side of the flags that follow
            __threadfence_system();
            const int32_t step = *cb.epoch + 1;
            for (int r = 0; r < cb.world; ++r)
                asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(cb.peer_flag[r]), "r"(step) : "memory");
            *cb.done = 0;
        }
    }
}

// ---- split-K over a thread-block cluster (dense form, few output tiles) ---------------------------
//
// A dense problem with fewer 128x256 tiles than SMs (decode-sized M, a single linear layer) would
// leave most of the GPU idle and stream the weights through a handful of SMs.  Here the S CTAs of a
// cluster share one output tile: CTA r accumulates K-blocks [r*KB/S, (r+1)*KB/S) in its own TMEM,
// then the partial tiles are exchanged through distributed shared memory -- CTA o owns columns
// [o*BN/S, (o+1)*BN/S) of the tile and receives every other CTA's partial of that band in the (by then
// idle) pipeline stages -- and each owner adds the S partials in rank order and stores bf16.  No
// workspace, no atomics, and the result does not depend on timing.  One tile per cluster.
//
// The exchange: a CTA stages the bands it does not own in its own shared memory (compact rows of BN/S floats,
// the 16-byte units of a row XOR-swizzled by the row number so that a lane per row stores without bank conflicts)
// and sends each to its owner as ONE bulk copy counted on the owner's barrier.  Stores or loads of the warps
// straight into another CTA's shared memory were measured first: with a lane per row every lane's 16 bytes cross
// the cluster network as a packet of their own, 0.2 to 0.4 us per warp instruction.
// Shared memory: S-1 staged and S-1 received bands of ceil32(live rows) x BN/S floats, up to 224 KB (S = 8, 256
// columns, 128 rows), so the barriers sit behind that area and not behind the pipeline stages.
constexpr int kSplitXchgBytes = 2 * 7 * kBlockM * (256 / 8) * 4;                 // 229,376
constexpr size_t kSplitSmemBytes = 1024 + kSplitXchgBytes + 256;
static_assert(kSplitSmemBytes <= 232448, "split-K exchange area exceeds the shared memory of an SM");
static_assert((size_t)Cfg<256>::kStages * (Cfg<256>::kStageBytes + Cfg<256>::kSfStage) <= kSplitXchgBytes &&
              (size_t)Cfg<128>::kStages * (Cfg<128>::kStageBytes + Cfg<128>::kSfStage) <= kSplitXchgBytes, "pipeline overlaps the barriers");

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
fp8_gemm_mx_splitk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA64,
                          const __grid_constant__ CUtensorMap tmA32, const __grid_constant__ CUtensorMap tmB,
                          const GemmParams p, const MxExtra x, const int S) {
    constexpr int kBN = Cfg<BN>::kBN, kStages = Cfg<BN>::kStages, kStageBytes = Cfg<BN>::kStageBytes;
    constexpr int kSfbBytes = Cfg<BN>::kSfbBytes, kSfStage = Cfg<BN>::kSfStage, kTxBytes = Cfg<BN>::kTxBytes;
    ptx::launch_dependents();      // the next kernel of the stream may come in under this one; it waits before it reads
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    uint8_t* sf_smem = smem + (size_t)kStages * kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSplitXchgBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = ptx::smem_u32(bars), bar_empty = ptx::smem_u32(bars + kStages);
    const uint32_t bar_tfull = ptx::smem_u32(bars + 2 * kStages);
    const uint32_t bar_xchg = ptx::smem_u32(bars + 2 * kStages + 1);       // the other CTAs' partials have arrived
    const uint32_t smem_tiles = ptx::smem_u32(smem), smem_sf = ptx::smem_u32(sf_smem);

    const uint32_t rank = ptx::cluster_ctarank();
    const int32_t cid = (int32_t)(blockIdx.x / (uint32_t)S);
    const int32_t m_blk = cid % p.num_m_blocks, n_blk = cid / p.num_m_blocks;
    const int32_t row0 = m_blk * kBlockM;
    const int32_t live = min(p.rows_total - row0, kBlockM);                 // the same in every CTA of the cluster
    const int32_t kbs = (p.num_k_blocks + S - 1) / S;
    const int32_t kb0 = (int32_t)rank * kbs, kb1 = min(p.num_k_blocks, kb0 + kbs);     // host guarantees kb0 < kb1
    const int W = kBN / S;                                                   // columns per owner (a multiple of 32)
    const uint32_t slot_bytes = (uint32_t)((live + 31) & ~31) * (uint32_t)W * 4u;    // one band: whole lane quarters of rows

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(bar_full + 8 * s, 1);
            ptx::mbar_init(bar_empty + 8 * s, 1);
        }
        ptx::mbar_init(bar_tfull, 1);
        ptx::mbar_init(bar_xchg, 1);
        ptx::mbar_arrive_expect_tx(bar_xchg, (uint32_t)(S - 1) * slot_bytes);
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

    if (warp == 0) {
        if (lane == 0) {
            ptx::prefetch_tensormap(&tmA);
            ptx::prefetch_tensormap(&tmA64);
            ptx::prefetch_tensormap(&tmA32);
            ptx::prefetch_tensormap(&tmB);
            WaitCtx w{abort_flag, p.status, 4};
            const uint8_t* sfa = x.sfa + (int64_t)m_blk * p.num_k_blocks * kSfaBytes;
            const uint8_t* sfb = x.sfb + (int64_t)(BN / 128) * n_blk * kSfaBytes;
            const CUtensorMap* tma = live <= 32 ? &tmA32 : (live <= 64 ? &tmA64 : &tmA);
            const uint32_t tx = (uint32_t)(kTxBytes - kABytes) + (live <= 32 ? 32u : (live <= 64 ? 64u : 128u)) * (uint32_t)kBlockK;
            // This grid may have been launched while the kernel before it still runs (programmatic stream serialisation).
            // The weights do not depend on it: the first ring-full of weight tiles and weight scales is requested at once;
            // the activations and their scales follow when that kernel's results are final.  A stage's barrier expects
            // all four copies from the start, so it completes only when the late ones have landed too.
            const int pre = min(kb1 - kb0, kStages);
            for (int i = 0; i < pre; ++i) {
                const uint32_t bar = bar_full + 8 * i;
                ptx::mbar_arrive_expect_tx(bar, tx);
                ptx::tma_load_2d(smem_tiles + i * kStageBytes + kABytes, &tmB, (kb0 + i) * kBlockK, n_blk * kBN, bar);
                ptx::bulk_load(smem_sf + i * kSfStage + kSfaBytes, sfb + (int64_t)(kb0 + i) * x.nb_pad * kSfaBytes, kSfbBytes, bar);
            }
            ptx::grid_dependency_wait();
            for (int i = 0; i < pre; ++i) {
                const uint32_t bar = bar_full + 8 * i;
                ptx::tma_load_2d(smem_tiles + i * kStageBytes, tma, (kb0 + i) * kBlockK, row0, bar);
                ptx::bulk_load(smem_sf + i * kSfStage, sfa + (int64_t)(kb0 + i) * kSfaBytes, kSfaBytes, bar);
            }
            uint32_t it = (uint32_t)pre;
            for (int kb = kb0 + pre; kb < kb1; ++kb, ++it) {
                const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                if (!wait_bar(bar_empty + 8 * s, ph ^ 1u, w)) break;
                const uint32_t bar = bar_full + 8 * s;
                ptx::mbar_arrive_expect_tx(bar, tx);
                const uint32_t dst = smem_tiles + s * kStageBytes;
                ptx::tma_load_2d(dst, tma, kb * kBlockK, row0, bar);
                ptx::tma_load_2d(dst + kABytes, &tmB, kb * kBlockK, n_blk * kBN, bar);
                const uint32_t sdst = smem_sf + s * kSfStage;
                ptx::bulk_load(sdst, sfa + (int64_t)kb * kSfaBytes, kSfaBytes, bar);
                ptx::bulk_load(sdst + kSfaBytes, sfb + (int64_t)kb * x.nb_pad * kSfaBytes, kSfbBytes, bar);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            WaitCtx w{abort_flag, p.status, 5};
            constexpr uint32_t idesc = ptx::umma_idesc_mx_e4m3(kBlockM, kBN, 0, 0);
            uint32_t it = 0;
            bool ok = true;
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                if (!wait_bar(bar_full + 8 * s, ph, w)) { ok = false; break; }
                ptx::tc_fence_after();
                const uint32_t a_addr = smem_tiles + s * kStageBytes;
                const uint32_t sf_addr = smem_sf + s * kSfStage;
                ptx::tmem_cp_32x128b_warpx4(tmem_base + kColSfa, ptx::umma_desc_sf(sf_addr));
                ptx::tmem_cp_32x128b_warpx4(tmem_base + kColSfb, ptx::umma_desc_sf(sf_addr + kSfaBytes));
                if (BN == 256)
                    ptx::tmem_cp_32x128b_warpx4(tmem_base + kColSfb + 4, ptx::umma_desc_sf(sf_addr + 2 * kSfaBytes));
                const uint64_t a_desc = ptx::umma_desc_k_sw128(a_addr);
                const uint64_t b_desc = ptx::umma_desc_k_sw128(a_addr + kABytes);
#pragma unroll
                for (int k = 0; k < kBlockK / 32; ++k)
                    ptx::mma_mxf8f6f4_block_scale(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, tmem_base + kColSfa,
                                                  tmem_base + kColSfb, (kb > kb0 || k > 0) ? 1u : 0u);
                ptx::mma_commit(bar_empty + 8 * s);
            }
            if (ok) ptx::mma_commit(bar_tfull);
        }
    } else {
        // all MMAs of this CTA have finished (and with them every read of the pipeline stages)
        WaitCtx w{abort_flag, p.status, 6};
        wait_bar(bar_tfull, 0u, w);
        ptx::tc_fence_after();
    }
    __syncwarp();
    // Every CTA of the cluster is done with its stages (they may now be overwritten) and has armed its exchange barrier.
    ptx::cluster_sync();

    // ---- exchange: the bands this CTA does not own are staged and sent; the two warps of a lane quarter take the even
    //      and the odd 32-column chunks of the row ----
    const uint32_t units = (uint32_t)W / 4u;                 // 16-byte units per staged row: 8, 16 or 32
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r_in_tile = quarter * 32 + lane;
    const uint32_t swz = (uint32_t)r_in_tile & (units - 1u);
    const bool quarter_live = warp >= 2 && quarter * 32 < live;     // warp-uniform: some row of this quarter holds data
    if (quarter_live) {
#pragma unroll 1
        for (int cc = half; cc < kBN / 32; cc += 2) {
            const int col = 32 * cc;
            const uint32_t o = (uint32_t)(col / W);
            if (o == rank) continue;
            uint32_t r[32];
            ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + col, r);
            ptx::tmem_ld_wait(r);
            const uint32_t send_slot = o < rank ? o : o - 1u;
            const uint32_t row_base = smem_tiles + send_slot * slot_bytes + (uint32_t)r_in_tile * (uint32_t)W * 4u;
            const uint32_t u0 = (uint32_t)(col % W) / 4u;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                ptx::st_shared_v4(row_base + (((u0 + (uint32_t)j) ^ swz) << 4), r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
        ptx::fence_proxy_async();                            // the staged rows are read by the bulk copies below
    }
    __syncthreads();
    if (threadIdx.x == 64) {
        for (uint32_t o = 0; o < (uint32_t)S; ++o) {
            if (o == rank) continue;
            const uint32_t send_slot = o < rank ? o : o - 1u, recv_slot = rank < o ? rank : rank - 1u;
            ptx::bulk_copy_to_cluster(ptx::mapa(smem_tiles + ((uint32_t)(S - 1) + recv_slot) * slot_bytes, o),
                                      smem_tiles + send_slot * slot_bytes, slot_bytes, ptx::mapa(bar_xchg, o));
        }
    }
    if (warp >= 2) {
        WaitCtx w{abort_flag, p.status, 7};
        wait_bar(bar_xchg, 0u, w);
    }

    // ---- the owned band: the S partials added in rank order (this CTA's own from tensor memory), bias, bf16 ----
    if (quarter_live) {
#pragma unroll 1
        for (int cc = half; cc < kBN / 32; cc += 2) {
            const int col = 32 * cc;
            if ((uint32_t)(col / W) != rank) continue;
            uint32_t r[32];
            ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + col, r);
            ptx::tmem_ld_wait(r);
            if (r_in_tile < live && *abort_flag == 0) {
                const int32_t n0 = n_blk * kBN + col;
                __nv_bfloat16* crow = p.C + (int64_t)(row0 + r_in_tile) * p.ldc + n0;
                const bool vec_ok = (reinterpret_cast<uintptr_t>(crow) & 15u) == 0;
                float f[32];
#pragma unroll
                for (int q = 0; q < 32; ++q) f[q] = 0.f;
                const uint32_t u0 = (uint32_t)(col % W) / 4u;
                for (uint32_t sl = 0; sl < (uint32_t)S; ++sl) {
                    if (sl == rank) {
#pragma unroll
                        for (int q = 0; q < 32; ++q) f[q] += __uint_as_float(r[q]);
                        continue;
                    }
                    const uint32_t recv_slot = sl < rank ? sl : sl - 1u;
                    const uint32_t row_base = smem_tiles + ((uint32_t)(S - 1) + recv_slot) * slot_bytes + (uint32_t)r_in_tile * (uint32_t)W * 4u;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float4 v = ptx::ld_shared_v4(row_base + (((u0 + (uint32_t)i) ^ swz) << 4));
                        f[4 * i + 0] += v.x; f[4 * i + 1] += v.y; f[4 * i + 2] += v.z; f[4 * i + 3] += v.w;
                    }
                }
                if (p.bias != nullptr) {
#pragma unroll
                    for (int q = 0; q < 32; ++q)
                        if (n0 + q < p.N) f[q] += __bfloat162float(p.bias[n0 + q]);
                }
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    if (n0 + j + 8 <= p.N && vec_ok) {
                        uint4 v;
                        v.x = pack_bf16x2(f[j + 0], f[j + 1]); v.y = pack_bf16x2(f[j + 2], f[j + 3]);
                        v.z = pack_bf16x2(f[j + 4], f[j + 5]); v.w = pack_bf16x2(f[j + 6], f[j + 7]);
                        *reinterpret_cast<uint4*>(crow + j) = v;
                    } else {
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            if (n0 + j + q < p.N) crow[j + q] = __float2bfloat16_rn(f[j + q]);
                    }
                }
            }
        }
    }

    ptx::tc_fence_before();
    __syncwarp();
    // No CTA leaves while a copy out of its shared memory may still be in flight: every owner has seen its barrier
    // complete, i.e. every copy into it has landed, before it arrives here.
    ptx::cluster_sync();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- CTA pairs: 256 x 256 output tiles on two SMs (cta_group::2), K split over the cluster ----------------
//
// The dense problems of a linear layer with a few hundred rows are bound by what an SM can pull from L2 per
// clock: a 128 x 256 tile moves 48 KB of operands per 128 of K.  Here two CTAs with consecutive cluster ranks share
// a 256 x 256 tile: each loads its own 128 rows of A and HALF of the tile's 256 weight rows (32 KB per 128 of K and
// SM), and one tcgen05.mma.cta_group::2 issued by the even CTA multiplies the pair's 256 rows by all 256 weight
// rows, reading the other half of B from the partner's shared memory; each CTA's tensor memory ends up with its
// own 128 x 256 accumulator.  Every copy is a plain 2-D tiled TMA load into the issuing CTA's own shared memory
// (no multicast); its bytes are counted on the even CTA's barrier, which the even CTA arms for both.  The scales
// travel as 2-D tiles too (the packed arrays seen as rows of 128 words): the CTA's own row block for A, both
// 128-column blocks for B, copied to tensor memory in both CTAs by one tcgen05.cp.cta_group::2.  The S K-slices
// of the cluster (S = 2 or 4; ranks 2k and 2k+1 form slice k) then reduce their partial tiles: slice k owns the
// k-th band of 256/S columns and receives the other slices' partials of that band in its shared memory.
struct PairCfg {
    static constexpr int kBN = 256;
    static constexpr int kStages = 6;
    static constexpr int kBHalf = (kBN / 2) * kBlockK;             // this CTA's half of the B tile
    static constexpr int kStageBytes = kABytes + kBHalf;           // 32 KB
    static constexpr int kSfStage = 512 + 512 * (kBN / 128);       // own A scale block, the tile's two B scale blocks
    static constexpr uint32_t kTxPair = 2u * (uint32_t)(kStageBytes + kSfStage);
    static constexpr size_t kSmemBytes = (size_t)kStages * (kStageBytes + kSfStage) + 1024 + 256;
    // the exchange reuses the pipeline stages: S-1 staged and S-1 received partial bands of 128 x 256/S floats
    static_assert(2 * 3 * kBlockM * (kBN / 4) * 4 <= kStages * kStageBytes && 2 * kBlockM * (kBN / 2) * 4 <= kStages * kStageBytes,
                  "partial bands do not fit the pipeline stages");
};

#ifdef KBN_TRACE
__device__ unsigned long long g_pair_trace[256][16];
#define KBN_PT(slot) do { if (lane == 0 && blockIdx.x < 256) g_pair_trace[blockIdx.x][slot] = trace_now(); } while (0)
#else
#define KBN_PT(slot) do { } while (0)
#endif

__global__ void __launch_bounds__(kThreads, 1)
fp8_gemm_mx_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmSfa, const __grid_constant__ CUtensorMap tmSfb, const GemmParams p,
                        const int32_t nb_pad, const int S) {
    constexpr int kStages = PairCfg::kStages, kStageBytes = PairCfg::kStageBytes, kSfStage = PairCfg::kSfStage, kBN = PairCfg::kBN;
    ptx::launch_dependents();      // the next kernel of the stream may come in under this one; it waits before it reads
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    uint8_t* sf_smem = smem + (size_t)kStages * kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sf_smem + (size_t)kStages * kSfStage);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = ptx::smem_u32(bars), bar_empty = ptx::smem_u32(bars + kStages);
    const uint32_t bar_tfull = ptx::smem_u32(bars + 2 * kStages);
    const uint32_t bar_xchg = ptx::smem_u32(bars + 2 * kStages + 1);       // the other slices' partials have arrived
    const uint32_t smem_tiles = ptx::smem_u32(smem), smem_sf = ptx::smem_u32(sf_smem);

    if (warp == 2) KBN_PT(0);
    const uint32_t rank = ptx::cluster_ctarank();
    const uint32_t pr = rank & 1u, ks = rank >> 1;          // place in the pair, K-slice
    const uint32_t leader = rank & ~1u;                      // the even CTA of the pair issues the MMAs
    const uint16_t pair_mask = (uint16_t)(3u << leader);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(bar_full + 8 * s, 1);             // armed by the even CTA's producer, bytes from both CTAs
            ptx::mbar_init(bar_empty + 8 * s, 1);            // one commit, delivered to both CTAs
        }
        ptx::mbar_init(bar_tfull, 1);
        ptx::mbar_init(bar_xchg, 1);
        ptx::mbar_arrive_expect_tx(bar_xchg, (uint32_t)(S - 1) * (uint32_t)(kBlockM * (kBN / S) * 4));
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), kTmemCols);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();           // the partner's barriers exist before anything is sent to them
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (warp == 2) KBN_PT(1);

    const int32_t cid = (int32_t)(blockIdx.x / (uint32_t)(2 * S));
    const int32_t m_pairs = (p.rows_total + 255) / 256;
    const int32_t m_pair = cid % m_pairs, n_blk = cid / m_pairs;
    const int32_t row0 = m_pair * 256 + (int32_t)pr * kBlockM;
    const int32_t live = max(0, min(p.rows_total - row0, kBlockM));
    const int32_t kbs = (p.num_k_blocks + S - 1) / S;
    const int32_t kb0 = (int32_t)ks * kbs, kb1 = min(p.num_k_blocks, kb0 + kbs);     // host guarantees kb0 < kb1

    if (warp == 0) {
        if (lane == 0) {
            ptx::prefetch_tensormap(&tmA);
            ptx::prefetch_tensormap(&tmB);
            ptx::prefetch_tensormap(&tmSfa);
            ptx::prefetch_tensormap(&tmSfb);
            WaitCtx w{abort_flag, p.status, 4};
            // The weights and their scales do not depend on the kernel before this one: the first ring-full is requested at
            // once.  The even CTA arms each stage's barrier for all eight copies of the pair, so a stage completes only
            // when the activations, requested after the wait below, have landed too.
            const int pre = min(kb1 - kb0, kStages);
            for (int i = 0; i < pre; ++i) {
                if (pr == 0) ptx::mbar_arrive_expect_tx(bar_full + 8 * i, PairCfg::kTxPair);
                const uint32_t bar = ptx::mapa(bar_full + 8 * i, leader);
                ptx::tma_load_2d_pair(smem_tiles + i * kStageBytes + kABytes, &tmB, (kb0 + i) * kBlockK, n_blk * kBN + (int32_t)pr * (kBN / 2), bar);
                ptx::tma_load_2d_pair(smem_sf + i * kSfStage + 512, &tmSfb, 0, (kb0 + i) * nb_pad + (kBN / 128) * n_blk, bar);
            }
            // results of the kernel before this one (the activations, the output buffer) are final from here on
            ptx::grid_dependency_wait();
            KBN_PT(2);
            for (int i = 0; i < pre; ++i) {
                const uint32_t bar = ptx::mapa(bar_full + 8 * i, leader);
                ptx::tma_load_2d_pair(smem_tiles + i * kStageBytes, &tmA, (kb0 + i) * kBlockK, row0, bar);
                ptx::tma_load_2d_pair(smem_sf + i * kSfStage, &tmSfa, 0, (row0 / kBlockM) * p.num_k_blocks + kb0 + i, bar);
            }
            uint32_t it = (uint32_t)pre;
            for (int kb = kb0 + pre; kb < kb1; ++kb, ++it) {
                const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                if (!wait_bar(bar_empty + 8 * s, ph ^ 1u, w)) break;
                if (pr == 0) ptx::mbar_arrive_expect_tx(bar_full + 8 * s, PairCfg::kTxPair);
                const uint32_t bar = ptx::mapa(bar_full + 8 * s, leader);
                const uint32_t dst = smem_tiles + s * kStageBytes;
                ptx::tma_load_2d_pair(dst, &tmA, kb * kBlockK, row0, bar);
                ptx::tma_load_2d_pair(dst + kABytes, &tmB, kb * kBlockK, n_blk * kBN + (int32_t)pr * (kBN / 2), bar);
                const uint32_t sdst = smem_sf + s * kSfStage;
                ptx::tma_load_2d_pair(sdst, &tmSfa, 0, (row0 / kBlockM) * p.num_k_blocks + kb, bar);
                ptx::tma_load_2d_pair(sdst + 512, &tmSfb, 0, kb * nb_pad + (kBN / 128) * n_blk, bar);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && pr == 0) {
            WaitCtx w{abort_flag, p.status, 5};
            constexpr uint32_t idesc = ptx::umma_idesc_mx_e4m3(256, kBN, 0, 0);
            uint32_t it = 0;
            bool ok = true;
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                if (!wait_bar(bar_full + 8 * s, ph, w)) { ok = false; break; }
                if (it == 0) KBN_PT(3);
                ptx::tc_fence_after();
                const uint32_t a_addr = smem_tiles + s * kStageBytes;
                const uint32_t sf_addr = smem_sf + s * kSfStage;
                ptx::tmem_cp_32x128b_warpx4_pair(tmem_base + kColSfa, ptx::umma_desc_sf(sf_addr));
                ptx::tmem_cp_32x128b_warpx4_pair(tmem_base + kColSfb, ptx::umma_desc_sf(sf_addr + 512));
                ptx::tmem_cp_32x128b_warpx4_pair(tmem_base + kColSfb + 4, ptx::umma_desc_sf(sf_addr + 1024));
                const uint64_t a_desc = ptx::umma_desc_k_sw128(a_addr);
                const uint64_t b_desc = ptx::umma_desc_k_sw128(a_addr + kABytes);
#pragma unroll
                for (int k = 0; k < kBlockK / 32; ++k)
                    ptx::mma_mxf8f6f4_block_scale_pair(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, tmem_base + kColSfa,
                                                       tmem_base + kColSfb, (kb > kb0 || k > 0) ? 1u : 0u);
                ptx::mma_commit_pair(bar_empty + 8 * s, pair_mask);
            }
            if (ok) ptx::mma_commit_pair(bar_tfull, pair_mask);
        }
    } else {
        // all MMAs of the pair have finished (and with them every read of the pipeline stages of both CTAs)
        WaitCtx w{abort_flag, p.status, 6};
        wait_bar(bar_tfull, 0u, w);
        ptx::tc_fence_after();
        if (warp == 2) KBN_PT(4);
    }
    __syncwarp();
    ptx::cluster_sync();          // every CTA of the cluster is done with its stages: they may now be overwritten
    if (warp == 2) KBN_PT(5);

    const int W = kBN / S;                                  // columns per owner
    {
        // ---- exchange: the partials of the column slices this CTA does not own are staged in its own shared memory
        //      (compact rows of W floats, 16-byte units XOR-swizzled by the row so that a lane per row stores without
        //      bank conflicts) and go to their owners -- the CTA of slice o in the same place of its pair -- as ONE bulk
        //      copy each, counted on the owner's barrier.  (Remote stores and remote loads from the warps were tried
        //      first: a strided 16-byte access per lane crosses the cluster network one small packet at a time, 0.2 to
        //      0.4 us per warp instruction.)  The CTA's own slice stays in tensor memory.  The two warps of a lane quarter
        //      take the even and the odd 32-column chunks of the row. ----
        const uint32_t slot_bytes = (uint32_t)(kBlockM * W * 4);
        const uint32_t units = (uint32_t)W / 4u;             // 16-byte units per staged row (32, 16 or 8... a power of two)
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int r_in_tile = quarter * 32 + lane;
        const uint32_t swz = (uint32_t)r_in_tile & (units - 1u);
        if (warp >= 2) {
#pragma unroll 1
            for (int cc = half; cc < kBN / 32; cc += 2) {
                const int col = 32 * cc;
                const uint32_t o = (uint32_t)(col / W);
                if (o == ks) continue;
                uint32_t r[32];
                ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + col, r);
                ptx::tmem_ld_wait(r);
                if (warp == 2) KBN_PT(8);
                const uint32_t send_slot = o < ks ? o : o - 1u;
                const uint32_t row_base = smem_tiles + send_slot * slot_bytes + (uint32_t)r_in_tile * (uint32_t)W * 4u;
                const uint32_t u0 = (uint32_t)(col % W) / 4u;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    ptx::st_shared_v4(row_base + (((u0 + (uint32_t)j) ^ swz) << 4), r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            }
            ptx::fence_proxy_async();                        // the staged rows are read by the bulk copies below
        }
        if (warp == 2) KBN_PT(9);
        __syncthreads();
        if (threadIdx.x == 64) {
            for (uint32_t o = 0; o < (uint32_t)S; ++o) {
                if (o == ks) continue;
                const uint32_t send_slot = o < ks ? o : o - 1u, recv_slot = ks < o ? ks : ks - 1u;
                const uint32_t owner = (o << 1) | pr;
                ptx::bulk_copy_to_cluster(ptx::mapa(smem_tiles + ((uint32_t)(S - 1) + recv_slot) * slot_bytes, owner),
                                          smem_tiles + send_slot * slot_bytes, slot_bytes, ptx::mapa(bar_xchg, owner));
            }
        }
        if (warp == 2) KBN_PT(10);
        if (warp >= 2) {
            WaitCtx w{abort_flag, p.status, 7};
            wait_bar(bar_xchg, 0u, w);
        }
        if (warp == 2) KBN_PT(6);
        // ---- the owned band: the S partials added in slice order (this CTA's own from tensor memory) ----
        if (warp >= 2 && quarter * 32 < live) {
#pragma unroll 1
            for (int cc = half; cc < kBN / 32; cc += 2) {
                const int col = 32 * cc;
                if ((uint32_t)(col / W) != ks) continue;
                uint32_t r[32];
                ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + col, r);
                ptx::tmem_ld_wait(r);
                if (r_in_tile < live && *abort_flag == 0) {
                    const int32_t n0 = n_blk * kBN + col;
                    __nv_bfloat16* crow = p.C + (int64_t)(row0 + r_in_tile) * p.ldc + n0;
                    const bool vec_ok = (reinterpret_cast<uintptr_t>(crow) & 15u) == 0;
                    float f[32];
#pragma unroll
                    for (int q = 0; q < 32; ++q) f[q] = 0.f;
                    const uint32_t u0 = (uint32_t)(col % W) / 4u;
                    for (uint32_t sl = 0; sl < (uint32_t)S; ++sl) {
                        if (sl == ks) {
#pragma unroll
                            for (int q = 0; q < 32; ++q) f[q] += __uint_as_float(r[q]);
                            continue;
                        }
                        const uint32_t recv_slot = sl < ks ? sl : sl - 1u;
                        const uint32_t row_base = smem_tiles + ((uint32_t)(S - 1) + recv_slot) * slot_bytes + (uint32_t)r_in_tile * (uint32_t)W * 4u;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float4 v = ptx::ld_shared_v4(row_base + (((u0 + (uint32_t)i) ^ swz) << 4));
                            f[4 * i + 0] += v.x; f[4 * i + 1] += v.y; f[4 * i + 2] += v.z; f[4 * i + 3] += v.w;
                        }
                    }
                    if (p.bias != nullptr) {
#pragma unroll
                        for (int q = 0; q < 32; ++q)
                            if (n0 + q < p.N) f[q] += __bfloat162float(p.bias[n0 + q]);
                    }
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        if (n0 + j + 8 <= p.N && vec_ok) {
                            uint4 v;
                            v.x = pack_bf16x2(f[j + 0], f[j + 1]); v.y = pack_bf16x2(f[j + 2], f[j + 3]);
                            v.z = pack_bf16x2(f[j + 4], f[j + 5]); v.w = pack_bf16x2(f[j + 6], f[j + 7]);
                            *reinterpret_cast<uint4*>(crow + j) = v;
                        } else {
#pragma unroll
                            for (int q = 0; q < 8; ++q)
                                if (n0 + j + q < p.N) crow[j + q] = __float2bfloat16_rn(f[j + q]);
                        }
                    }
                }
            }
        }
        if (warp >= 2) ptx::tc_fence_before();
        if (warp == 2) KBN_PT(11);
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 2) KBN_PT(12);
    ptx::cluster_sync();          // neither CTA of a pair frees tensor memory while the other still reads its own
    if (warp == 2) KBN_PT(7);
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

// ---- scale packing -----------------------------------------------------------------------------

__device__ __forceinline__ uint32_t ue8m0_word(float s) {
    uint32_t b = (__float_as_uint(s) >> 23) & 0xffu;
    return b * 0x01010101u;
}

// fp32 per-row scales (any strides) -> packed blocks [row_blocks][KB][32][4] words; rows past the end get 1.0
__global__ void pack_sf_rows_kernel(const float* __restrict__ s, int64_t rows, int KB, int64_t s_row, int64_t s_grp,
                                    uint32_t* __restrict__ out, int64_t total_words) {
    const int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (w >= total_words) return;
    const int i = (int)(w & 3), l = (int)((w >> 2) & 31);
    const int64_t blk_kb = w >> 7;
    const int kb = (int)(blk_kb % KB);
    const int64_t row = (blk_kb / KB) * 128 + i * 32 + l;
    out[w] = row < rows ? ue8m0_word(s[row * s_row + kb * s_grp]) : 0x7f7f7f7fu;
}

// fp32 128x128 block scales [E][NB][KB] -> packed [E][KB][nb_pad][128 words], every word of a block equal
__global__ void pack_sf_weights_kernel(const float* __restrict__ sb, int E, int NB, int KB, int nb_pad,
                                       uint32_t* __restrict__ out, int64_t total_words) {
    const int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (w >= total_words) return;
    const int64_t blk = w >> 7;
    const int nb = (int)(blk % nb_pad);
    const int64_t ek = blk / nb_pad;
    const int kb = (int)(ek % KB);
    const int e = (int)(ek / KB);
    out[w] = nb < NB ? ue8m0_word(sb[((int64_t)e * NB + nb) * KB + kb]) : 0x7f7f7f7fu;
}

// Counts scales that are not positive powers of two (mantissa bits set, zero, negative, inf/nan).
__global__ void count_non_pow2_kernel(const float* __restrict__ s, int64_t n, int32_t* __restrict__ count) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t b = __float_as_uint(s[i]);
    const uint32_t e = (b >> 23) & 0xffu;
    if ((b & 0x807fffffu) != 0u || e == 0u || e == 255u) atomicAdd(count, 1);
}

// ---- host side -----------------------------------------------------------------------------------

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

// Encoded tensor maps of this thread's recent calls.  A map depends on nothing but the arguments it was encoded from
// (address, extents, box, promotion), so an entry stays valid whatever happens to the memory behind the address; a
// layer that calls the same GEMM on the same buffers every step pays for the driver's encoder once per operand.
struct TmapCacheEntry {
    const void* base = nullptr;
    int64_t rows = 0, K = 0;
    int32_t box_rows = 0, kind = 0;      // kind: L2 promotion for operand maps, -1 for scale maps
    CUtensorMap tm;
};
constexpr int kTmapCacheSize = 64;
static TmapCacheEntry* tmap_cache_slot(const void* base, int64_t rows, int64_t K, int box_rows, int kind, bool* hit) {
    static thread_local TmapCacheEntry cache[kTmapCacheSize];
    uint64_t h = reinterpret_cast<uintptr_t>(base) >> 4;
    h = (h ^ (h >> 17) ^ (uint64_t)rows * 0x9e3779b97f4a7c15ull ^ (uint64_t)K * 0xc2b2ae3d27d4eb4full ^ (uint64_t)(box_rows * 8 + kind + 1)) * 0xff51afd7ed558ccdull;
    TmapCacheEntry* e = &cache[(h >> 40) % kTmapCacheSize];
    *hit = e->base == base && e->rows == rows && e->K == K && e->box_rows == box_rows && e->kind == kind;
    return e;
}

static int make_tmap(CUtensorMap* tm, const void* base, int64_t rows, int64_t K, int box_rows, CUtensorMapL2promotion promo) {
    bool hit = false;
    TmapCacheEntry* ce = tmap_cache_slot(base, rows, K, box_rows, (int)promo, &hit);
    if (hit) {
        *tm = ce->tm;
        return KBN_OK;
    }
    EncodeTiledFn fn = encode_fn();
    KBN_REQUIRE(fn, KBN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K};
    cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    KBN_REQUIRE(r == CUDA_SUCCESS, KBN_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld K=%lld)",
                (int)r, (long long)rows, (long long)K);
    ce->base = base; ce->rows = rows; ce->K = K; ce->box_rows = box_rows; ce->kind = (int)promo;
    ce->tm = *tm;
    return KBN_OK;
}

// Packed scale array seen as rows of 128 32-bit words (one 512-byte scale block per row): boxes of `box_rows` blocks.
static int make_tmap_sf(CUtensorMap* tm, const void* base, int64_t blocks, int box_rows) {
    bool hit = false;
    TmapCacheEntry* ce = tmap_cache_slot(base, blocks, 128, box_rows, -1, &hit);
    if (hit) {
        *tm = ce->tm;
        return KBN_OK;
    }
    EncodeTiledFn fn = encode_fn();
    KBN_REQUIRE(fn, KBN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {128, (cuuint64_t)blocks};
    cuuint64_t strides[1] = {512};
    cuuint32_t box[2] = {128, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    KBN_REQUIRE(r == CUDA_SUCCESS, KBN_ERR_CUDA, "cuTensorMapEncodeTiled (scales) failed with CUresult %d (blocks=%lld)", (int)r, (long long)blocks);
    ce->base = base; ce->rows = blocks; ce->K = 128; ce->box_rows = box_rows; ce->kind = -1;
    ce->tm = *tm;
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
        KBN_CUDA(cudaFuncSetAttribute(fp8_gemm_mx_kernel<256, kEpiStore, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<256>::kSmemBytes));
        KBN_CUDA(cudaFuncSetAttribute(fp8_gemm_mx_kernel<256, kEpiAct, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<256>::kSmemBytes));
        KBN_CUDA(cudaFuncSetAttribute(fp8_gemm_mx_kernel<256, kEpiCombine, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<256>::kSmemBytes));
        KBN_CUDA(cudaFuncSetAttribute(fp8_gemm_mx_kernel<128, kEpiStore, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<128>::kSmemBytes));
        KBN_CUDA(cudaFuncSetAttribute(fp8_gemm_mx_kernel<256, kEpiStore, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSwapSmemBytes));
        KBN_CUDA(cudaFuncSetAttribute(fp8_gemm_mx_kernel<256, kEpiAct, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSwapSmemBytes));
        KBN_CUDA(cudaFuncSetAttribute(fp8_gemm_mx_kernel<256, kEpiCombine, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSwapSmemBytes));
        KBN_CUDA(cudaFuncSetAttribute(fp8_gemm_mx_splitk_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSplitSmemBytes));
        KBN_CUDA(cudaFuncSetAttribute(fp8_gemm_mx_splitk_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSplitSmemBytes));
        KBN_CUDA(cudaFuncSetAttribute(fp8_gemm_mx_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PairCfg::kSmemBytes));
        ok[dev] = 1;
    }
    return KBN_OK;
}

static inline int32_t cdiv32(int64_t a, int64_t b) { return (int32_t)((a + b - 1) / b); }

// Clusters of `split` CTAs of the split-K kernel that can be resident at once (cached per device).
template <int BN>
static int max_active_clusters(int split) {
    static int cache[64][9] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || split < 2 || split > 8) return 0;
    if (cache[dev][split] == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(split * 64));
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kSplitSmemBytes;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)split;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, fp8_gemm_mx_splitk_kernel<BN>, &cfg) != cudaSuccess) {
            cudaGetLastError();
            n = -1;
        }
        cache[dev][split] = n > 0 ? n : -1;
    }
    return cache[dev][split] > 0 ? cache[dev][split] : 0;
}

// Clusters of 2*S CTAs of the CTA-pair kernel that can be resident at once (cached per device).
static int max_active_pair_clusters(int S) {
    static int cache[64][5] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || S < 2 || S > 4) return 0;
    if (cache[dev][S] == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(2 * S * 16));
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = PairCfg::kSmemBytes;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)(2 * S);
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, fp8_gemm_mx_pair_kernel, &cfg) != cudaSuccess) {
            cudaGetLastError();
            n = -1;
        }
        cache[dev][S] = n > 0 ? n : -1;
    }
    return cache[dev][S] > 0 ? cache[dev][S] : 0;
}

// K-slices per cluster of the CTA-pair kernel for a dense problem, 0 when the problem does not suit it: more than one
// row block, too few 256 x 256 tiles to give every SM one, and a split that puts a CTA on at least three SMs in five
// with every cluster resident at once.
static int pair_plan(const GemmParams& p) {
    if (p.mode != kDense || p.rows_total <= kBlockM || p.N <= 128 || p.K % 128 != 0) return 0;
    const int64_t pair_tiles = (int64_t)cdiv32(p.rows_total, 256) * cdiv32(p.N, PairCfg::kBN);
    for (int S = 4; S >= 2; S /= 2) {
        const int kbs = (p.num_k_blocks + S - 1) / S;
        if (2 * S * pair_tiles > sm_count() || (S - 1) * kbs >= p.num_k_blocks || p.num_k_blocks < 2 * S) continue;
        if (pair_tiles > max_active_pair_clusters(S)) continue;
        return 2 * S * pair_tiles * 5 >= (int64_t)sm_count() * 3 ? S : 0;
    }
    return 0;
}

static int launch_pair(const void* A, int64_t a_rows, const void* B, int64_t b_rows, const GemmParams& p, const void* sfa, const void* sfb,
                       int S, cudaStream_t st) {
    constexpr int BN = PairCfg::kBN;
    CUtensorMap tmA, tmB, tmSfa, tmSfb;
    int rc = make_tmap(&tmA, A, a_rows, p.K, kBlockM, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    if (rc != KBN_OK) return rc;
    rc = make_tmap(&tmB, B, b_rows, p.K, BN / 2, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != KBN_OK) return rc;
    const int32_t nb_pad = (cdiv32(p.N, 128) + 1) / 2 * 2;
    rc = make_tmap_sf(&tmSfa, sfa, (int64_t)cdiv32(p.rows_total, kBlockM) * p.num_k_blocks, 1);
    if (rc != KBN_OK) return rc;
    rc = make_tmap_sf(&tmSfb, sfb, (int64_t)p.num_k_blocks * nb_pad, BN / 128);
    if (rc != KBN_OK) return rc;
    const int64_t pair_tiles = (int64_t)cdiv32(p.rows_total, 256) * cdiv32(p.N, BN);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(pair_tiles * 2 * S));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = PairCfg::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)(2 * S);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    KBN_CUDA(cudaLaunchKernelEx(&cfg, fp8_gemm_mx_pair_kernel, tmA, tmB, tmSfa, tmSfb, p, nb_pad, S));
    KBN_CHECK_LAUNCH();
    return KBN_OK;
}

template <int BN>
static int launch_splitk(const CUtensorMap& tmA, const CUtensorMap& tmA64, const CUtensorMap& tmA32, const CUtensorMap& tmB,
                         const GemmParams& p, const MxExtra& x, int split, int64_t tiles, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles * split));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSplitSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)split;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    KBN_CUDA(cudaLaunchKernelEx(&cfg, fp8_gemm_mx_splitk_kernel<BN>, tmA, tmA64, tmA32, tmB, p, x, split));
    KBN_CHECK_LAUNCH();
    return KBN_OK;
}

// m_blocks_upper: number of 128-row blocks (an upper bound in the masked form).
// act: fused activation epilogue (p.act_* filled in, p.N = output columns, B has 2*p.N rows per expert).
// combine: epilogue that sends the rows to their source ranks (masked form, 256-wide tiles).
// hooks: the expert-parallel layer's ties to its neighbouring kernels (see EpHooks); with them the kernel is launched
// with programmatic stream serialisation, i.e. it may start while the kernel before it in the stream still runs.
static int launch(const void* A, int64_t a_rows, const void* B, int64_t b_rows, GemmParams& p, const void* sfa, const void* sfb,
                  int64_t m_blocks_upper, cudaStream_t st, bool act = false, const CombineEpilogue* combine = nullptr,
                  const EpHooks* hooks = nullptr) {
    int rc = check_device();
    if (rc != KBN_OK) return rc;
    KBN_REQUIRE(sfa && sfb, KBN_ERR_ARG, "fp8 gemm (ue8m0): null packed scales");
    KBN_REQUIRE(aligned16(A) && aligned16(B) && aligned16(sfa) && aligned16(sfb), KBN_ERR_ARG, "fp8 gemm (ue8m0): pointers must be 16-byte aligned");
    KBN_REQUIRE(p.K % 16 == 0 && p.K > 0 && p.N > 0, KBN_ERR_ARG, "fp8 gemm (ue8m0): K=%d must be a positive multiple of 16", p.K);
    KBN_REQUIRE(a_rows < (1ll << 31) && b_rows < (1ll << 31), KBN_ERR_ARG, "fp8 gemm (ue8m0): more than 2^31 rows");
    // a few hundred rows of a dense layer: 256 x 256 tiles on CTA pairs
    if (!act && !combine && !hooks) {
        const int S = pair_plan(p);
        if (S > 0) {
            rc = gemm_status_ptr(&p.status);
            if (rc != KBN_OK) return rc;
            return launch_pair(A, a_rows, B, b_rows, p, sfa, sfb, S, st);
        }
    }
    // 256-wide tiles unless that would leave SMs without a tile and 128-wide tiles fill more of them
    int bn = 256;
    if (p.mode != kMasked && p.N > 128 && m_blocks_upper * cdiv32(p.N, 256) < sm_count()) bn = 128;
    // Dense problems with so few tiles that at least half of the SMs would idle: split K over a cluster
    // (the widest split whose clusters are all resident at once and leave every CTA some K-blocks).
    int split = 1;
    if (p.mode == kDense) {
        const int bn_s = p.N > 128 ? 256 : 128;
        const int64_t tiles_s = m_blocks_upper * cdiv32(p.N, bn_s);
        for (int s2 = bn_s == 256 ? 8 : 4; s2 >= 2; s2 /= 2) {
            const int kbs = (p.num_k_blocks + s2 - 1) / s2;
            if (tiles_s * s2 > sm_count() || (s2 - 1) * kbs >= p.num_k_blocks || p.num_k_blocks < 2 * s2) continue;
            const int resident = bn_s == 256 ? max_active_clusters<256>(s2) : max_active_clusters<128>(s2);
            if (tiles_s > resident) continue;
            split = s2;
            bn = bn_s;
            break;
        }
    }
    if (act || combine) {           // act: 128 output columns (= 256 weight rows) per tile
        bn = 256;
        split = 1;
    }
    p.num_n_blocks = act ? cdiv32(p.N, 128) : cdiv32(p.N, bn);
    const int64_t max_tiles = m_blocks_upper * p.num_n_blocks;
    CUtensorMap tmA, tmA64, tmA32, tmB;
    rc = make_tmap(&tmA, A, a_rows, p.K, kBlockM, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    if (rc != KBN_OK) return rc;
    rc = make_tmap(&tmA64, A, a_rows, p.K, 64, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    if (rc != KBN_OK) return rc;
    rc = make_tmap(&tmA32, A, a_rows, p.K, 32, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    if (rc != KBN_OK) return rc;
    rc = make_tmap(&tmB, B, b_rows, p.K, act ? 128 : bn, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != KBN_OK) return rc;
    rc = gemm_status_ptr(&p.status);
    if (rc != KBN_OK) return rc;
    MxExtra x;
    x.sfa = static_cast<const uint8_t*>(sfa);
    x.sfb = static_cast<const uint8_t*>(sfb);
    x.nb_pad = (cdiv32(act ? 2 * (int64_t)p.N : p.N, 128) + 1) / 2 * 2;
    int64_t grid = sm_count();
    if (max_tiles < grid) grid = max_tiles;
    if (grid <= 0) return KBN_OK;
    CombineEpilogue cb{};
    if (combine) cb = *combine;
    EpHooks hk{};
    if (hooks) hk = *hooks;
    if (split > 1)
        return bn == 256 ? launch_splitk<256>(tmA, tmA64, tmA32, tmB, p, x, split, max_tiles, st)
                         : launch_splitk<128>(tmA, tmA64, tmA32, tmB, p, x, split, max_tiles, st);
    // masked layout with at most 256 rows per expert (decode batches): the operands trade places, see the kernel.
    // A caller that knows its load says so: above about 56 expected rows per expert many blocks have more than 64 live
    // rows, and those are faster in the plain order.
    const bool swap = p.mode == kMasked && p.max_m <= 256 && bn == 256 && (p.expected_m <= 0 || p.expected_m <= kSwapMaxExpectedRows);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(hk.sched != nullptr ? kThreadsMain : kThreads);      // the scheduler warp only where tiles come from a counter
    cfg.dynamicSmemBytes = swap ? kSwapSmemBytes : (bn == 256 ? Cfg<256>::kSmemBytes : Cfg<128>::kSmemBytes);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (hooks || p.mode == kDense) ? 1 : 0;
    auto go = [&](auto kernel) { return cudaLaunchKernelEx(&cfg, kernel, tmA, tmA64, tmA32, tmB, p, x, cb, hk); };
    cudaError_t le;
    if (swap && combine) le = go(fp8_gemm_mx_kernel<256, kEpiCombine, true>);
    else if (swap && act) le = go(fp8_gemm_mx_kernel<256, kEpiAct, true>);
    else if (swap) le = go(fp8_gemm_mx_kernel<256, kEpiStore, true>);
    else if (combine) le = go(fp8_gemm_mx_kernel<256, kEpiCombine, false>);
    else if (act) le = go(fp8_gemm_mx_kernel<256, kEpiAct, false>);
    else if (bn == 256) le = go(fp8_gemm_mx_kernel<256, kEpiStore, false>);
    else le = go(fp8_gemm_mx_kernel<128, kEpiStore, false>);
    KBN_CUDA(le);
    KBN_CHECK_LAUNCH();
    return KBN_OK;
}

static void fill_params(GemmParams& p, void* C, int64_t ldc, int64_t rows, int64_t N, int64_t K, int64_t E, int64_t max_m, int mode) {
    p.sa = nullptr; p.sb = nullptr; p.bias = nullptr; p.sa_exp = p.sa_row = p.sa_grp = 0;
    p.C = static_cast<__nv_bfloat16*>(C); p.ldc = ldc;
    p.rows_total = (int32_t)rows; p.N = (int32_t)N; p.K = (int32_t)K; p.E = (int32_t)E; p.max_m = (int32_t)max_m;
    p.num_m_blocks = mode == kMasked ? 0 : cdiv32(rows, kBlockM);
    p.num_n_blocks = 0 /* set by launch() */; p.num_k_blocks = cdiv32(K, kBlockK); p.sb_nb = cdiv32(N, 128);
    p.mode = mode;
}

}  // namespace mx
}  // namespace kbn

#ifdef KBN_TRACE
extern "C" int kbn_debug_pair_trace(unsigned long long* host_out) {
    using namespace kbn;
    KBN_CUDA(cudaDeviceSynchronize());
    KBN_CUDA(cudaMemcpyFromSymbol(host_out, mx::g_pair_trace, sizeof(unsigned long long) * 256 * 16));
    return KBN_OK;
}
#endif

extern "C" int64_t kbn_packed_sf_rows_bytes(int64_t rows, int64_t K) {
    return ((rows + 127) / 128) * ((K + 127) / 128) * 512;
}

extern "C" int64_t kbn_packed_sf_weights_bytes(int64_t E, int64_t N, int64_t K) {
    int64_t nb_pad = ((N + 127) / 128 + 1) / 2 * 2;
    return E * ((K + 127) / 128) * nb_pad * 512;
}

extern "C" int kbn_pack_sf_rows(const float* scale, int64_t rows, int64_t K, int64_t s_row, int64_t s_grp, void* packed,
                                kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(rows >= 0 && K >= 0, KBN_ERR_ARG, "kbn_pack_sf_rows: negative size");
    const int64_t words = kbn_packed_sf_rows_bytes(rows, K) / 4;
    if (words == 0) return KBN_OK;
    KBN_REQUIRE(scale && packed && aligned16(packed), KBN_ERR_ARG, "kbn_pack_sf_rows: null or misaligned pointer");
    mx::pack_sf_rows_kernel<<<(unsigned)((words + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        scale, rows, (int)((K + 127) / 128), s_row, s_grp, static_cast<uint32_t*>(packed), words);
    KBN_CHECK_LAUNCH();
    return KBN_OK;
}

extern "C" int kbn_pack_sf_weights(const float* sb, int64_t E, int64_t N, int64_t K, void* packed, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(E >= 0 && N >= 0 && K >= 0, KBN_ERR_ARG, "kbn_pack_sf_weights: negative size");
    const int64_t words = kbn_packed_sf_weights_bytes(E, N, K) / 4;
    if (words == 0) return KBN_OK;
    KBN_REQUIRE(sb && packed && aligned16(packed), KBN_ERR_ARG, "kbn_pack_sf_weights: null or misaligned pointer");
    const int NB = (int)((N + 127) / 128);
    mx::pack_sf_weights_kernel<<<(unsigned)((words + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        sb, (int)E, NB, (int)((K + 127) / 128), (NB + 1) / 2 * 2, static_cast<uint32_t*>(packed), words);
    KBN_CHECK_LAUNCH();
    return KBN_OK;
}

extern "C" int kbn_count_non_pow2_scales(const float* s, int64_t n, int32_t* device_count, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(n >= 0, KBN_ERR_ARG, "kbn_count_non_pow2_scales: negative size");
    KBN_REQUIRE(device_count, KBN_ERR_ARG, "kbn_count_non_pow2_scales: null pointer");
    if (n == 0) return KBN_OK;
    KBN_REQUIRE(s, KBN_ERR_ARG, "kbn_count_non_pow2_scales: null pointer");
    mx::count_non_pow2_kernel<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(s, n, device_count);
    KBN_CHECK_LAUNCH();
    return KBN_OK;
}

extern "C" int kbn_fp8_gemm_nt_ue8m0(const void* A, const void* sfa_packed, const void* B, const void* sfb_packed, const void* bias,
                                     void* C, int64_t ldc, int64_t M, int64_t N, int64_t K, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(M >= 0 && N >= 0 && K >= 0, KBN_ERR_ARG, "kbn_fp8_gemm_nt_ue8m0: negative size");
    if (M == 0 || N == 0) return KBN_OK;
    KBN_REQUIRE(A && B && C && ldc >= N, KBN_ERR_ARG, "kbn_fp8_gemm_nt_ue8m0: null pointer or ldc < N");
    GemmParams p{};
    mx::fill_params(p, C, ldc, M, N, K, 1, 0, kDense);
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    return mx::launch(A, M, B, N, p, sfa_packed, sfb_packed, p.num_m_blocks, static_cast<cudaStream_t>(stream));
}

extern "C" int kbn_fp8_grouped_gemm_contig_ue8m0(const void* A, const void* sfa_packed, const void* B, const void* sfb_packed,
                                                 void* C, int64_t ldc, const int32_t* row_expert, int64_t M_sum, int64_t N,
                                                 int64_t K, int64_t E, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(M_sum >= 0 && N >= 0 && K >= 0 && E >= 0, KBN_ERR_ARG, "kbn_fp8_grouped_gemm_contig_ue8m0: negative size");
    if (M_sum == 0 || N == 0 || E == 0) return KBN_OK;
    KBN_REQUIRE(A && B && C && row_expert && ldc >= N, KBN_ERR_ARG, "kbn_fp8_grouped_gemm_contig_ue8m0: null pointer or ldc < N");
    KBN_REQUIRE(E * N < (1ll << 31), KBN_ERR_ARG, "kbn_fp8_grouped_gemm_contig_ue8m0: E*N too large");
    GemmParams p{};
    mx::fill_params(p, C, ldc, M_sum, N, K, E, 0, kContig);
    p.row_expert = row_expert;
    return mx::launch(A, M_sum, B, E * N, p, sfa_packed, sfb_packed, p.num_m_blocks, static_cast<cudaStream_t>(stream));
}

extern "C" int kbn_fp8_grouped_gemm_masked_ue8m0(const void* A, const void* sfa_packed, const void* B, const void* sfb_packed,
                                                 void* C, const int32_t* masked_m, int64_t E, int64_t max_m, int64_t N, int64_t K,
                                                 kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(E >= 0 && max_m >= 0 && N >= 0 && K >= 0, KBN_ERR_ARG, "kbn_fp8_grouped_gemm_masked_ue8m0: negative size");
    if (E == 0 || max_m == 0 || N == 0) return KBN_OK;
    KBN_REQUIRE(A && B && C && masked_m, KBN_ERR_ARG, "kbn_fp8_grouped_gemm_masked_ue8m0: null pointer");
    KBN_REQUIRE(max_m % 128 == 0, KBN_ERR_ARG, "kbn_fp8_grouped_gemm_masked_ue8m0: max_m=%lld must be a multiple of 128", (long long)max_m);
    KBN_REQUIRE(E * N < (1ll << 31) && E * max_m < (1ll << 31), KBN_ERR_ARG, "kbn_fp8_grouped_gemm_masked_ue8m0: too large");
    GemmParams p{};
    mx::fill_params(p, C, N, E * max_m, N, K, E, max_m, kMasked);
    p.masked_m = masked_m;
    return mx::launch(A, E * max_m, B, E * N, p, sfa_packed, sfb_packed, E * ((max_m + 127) / 128), static_cast<cudaStream_t>(stream));
}

// ---- masked grouped GEMM2 whose epilogue returns the rows to their source ranks -------------------

namespace kbn {
namespace mx {

// Not part of the C ABI: called by the expert-parallel layer, which owns the peer mappings.
int gemm_masked_ue8m0_combine(const void* A, const void* sfa_packed, const void* B, const void* sfb_packed, const int32_t* masked_m,
                              int64_t E, int64_t max_m, int64_t N, int64_t K, const CombineEpilogue& cb, int64_t expected_m,
                              const EpHooks* hooks, cudaStream_t st) {
    const char* who = "fp8 gemm (ue8m0, combine epilogue)";
    KBN_REQUIRE(E > 0 && max_m > 0 && N > 0 && K > 0 && A && B && masked_m, KBN_ERR_ARG, "%s: bad arguments", who);
    KBN_REQUIRE(max_m % 128 == 0 && N % 32 == 0, KBN_ERR_ARG, "%s: max_m must be a multiple of 128 and N of 32", who);
    KBN_REQUIRE(E * N < (1ll << 31) && E * max_m < (1ll << 31), KBN_ERR_ARG, "%s: too large", who);
    KBN_REQUIRE(cb.world >= 0 && cb.world <= kMaxPeerRanks && cb.meta && cb.done && cb.epoch, KBN_ERR_ARG, "%s: bad peer description", who);
    GemmParams p{};
    fill_params(p, nullptr, N, E * max_m, N, K, E, max_m, kMasked);
    p.masked_m = masked_m;
    p.expected_m = (int32_t)std::min<int64_t>(std::max<int64_t>(expected_m, 0), 1 << 30);
    // the grid is never empty here: the last CTA must signal the peers even when no expert has rows
    return launch(A, E * max_m, B, E * N, p, sfa_packed, sfb_packed, E * (max_m / 128), st, false, &cb, hooks);
}

}  // namespace mx
}  // namespace kbn

// ---- grouped GEMM1 with the activation in the epilogue ------------------------------------------

namespace kbn {
namespace mx {

static int fill_act(GemmParams& p, const char* who, void* q, int64_t ld_q, float* scale, int64_t s_row, int64_t s_grp, void* sf_packed,
                    int64_t I, cudaStream_t st) {
    KBN_REQUIRE(q && scale, KBN_ERR_ARG, "%s: null output pointer", who);
    KBN_REQUIRE(I % 128 == 0, KBN_ERR_ARG, "%s: I=%lld must be a multiple of 128", who, (long long)I);
    KBN_REQUIRE(ld_q >= I && ld_q % 16 == 0 && aligned16(q), KBN_ERR_ARG, "%s: q must be 16-byte aligned with a row stride that is a multiple of 16", who);
    KBN_REQUIRE(!sf_packed || aligned16(sf_packed), KBN_ERR_ARG, "%s: packed scales must be 16-byte aligned", who);
    p.act_q = static_cast<uint8_t*>(q);
    p.act_ld = ld_q;
    p.act_scale = scale;
    p.act_s_row = s_row;
    p.act_s_grp = s_grp;
    p.act_packed = static_cast<uint32_t*>(sf_packed);
    return silu_table_for_stream(st, &p.act_table);
}

}  // namespace mx
}  // namespace kbn

extern "C" int kbn_fp8_grouped_gemm_contig_ue8m0_silu(const void* A, const void* sfa_packed, const void* W13, const void* sfb_packed,
                                                      void* q, int64_t ld_q, float* scale, int64_t s_row, int64_t s_grp, void* sf_packed,
                                                      const int32_t* row_expert, int64_t M_sum, int64_t I, int64_t K, int64_t E,
                                                      kbn_stream_t stream) {
    using namespace kbn;
    const char* who = "kbn_fp8_grouped_gemm_contig_ue8m0_silu";
    KBN_REQUIRE(M_sum >= 0 && I >= 0 && K >= 0 && E >= 0, KBN_ERR_ARG, "%s: negative size", who);
    if (M_sum == 0 || I == 0 || E == 0) return KBN_OK;
    KBN_REQUIRE(A && W13 && row_expert, KBN_ERR_ARG, "%s: null pointer", who);
    KBN_REQUIRE(E * 2 * I < (1ll << 31), KBN_ERR_ARG, "%s: E*2*I too large", who);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    GemmParams p{};
    mx::fill_params(p, nullptr, 0, M_sum, I, K, E, 0, kContig);
    p.row_expert = row_expert;
    int rc = mx::fill_act(p, who, q, ld_q, scale, s_row, s_grp, sf_packed, I, st);
    if (rc != KBN_OK) return rc;
    return mx::launch(A, M_sum, W13, E * 2 * I, p, sfa_packed, sfb_packed, p.num_m_blocks, st, true);
}

namespace kbn {
namespace mx {
// The masked GEMM1 + activation with the caller's expected rows per expert (0: unknown), which picks the operand order.
int gemm1_masked_ue8m0_silu(const void* A, const void* sfa_packed, const void* W13, const void* sfb_packed, void* q, float* scale,
                            void* sf_packed, const int32_t* masked_m, int64_t E, int64_t max_m, int64_t I, int64_t K, int64_t expected_m,
                            const EpHooks* hooks, cudaStream_t st) {
    const char* who = "kbn_fp8_grouped_gemm_masked_ue8m0_silu";
    KBN_REQUIRE(E >= 0 && max_m >= 0 && I >= 0 && K >= 0, KBN_ERR_ARG, "%s: negative size", who);
    if (E == 0 || max_m == 0 || I == 0) return KBN_OK;
    KBN_REQUIRE(A && W13 && masked_m, KBN_ERR_ARG, "%s: null pointer", who);
    KBN_REQUIRE(max_m % 128 == 0, KBN_ERR_ARG, "%s: max_m=%lld must be a multiple of 128", who, (long long)max_m);
    KBN_REQUIRE(E * 2 * I < (1ll << 31) && E * max_m < (1ll << 31), KBN_ERR_ARG, "%s: too large", who);
    GemmParams p{};
    fill_params(p, nullptr, 0, E * max_m, I, K, E, max_m, kMasked);
    p.masked_m = masked_m;
    p.expected_m = (int32_t)std::min<int64_t>(std::max<int64_t>(expected_m, 0), 1 << 30);
    int rc = fill_act(p, who, q, I, scale, I / 128, 1, sf_packed, I, st);
    if (rc != KBN_OK) return rc;
    return launch(A, E * max_m, W13, E * 2 * I, p, sfa_packed, sfb_packed, E * (max_m / 128), st, true, nullptr, hooks);
}
}  // namespace mx
}  // namespace kbn

extern "C" int kbn_fp8_grouped_gemm_masked_ue8m0_silu(const void* A, const void* sfa_packed, const void* W13, const void* sfb_packed,
                                                      void* q, float* scale, void* sf_packed, const int32_t* masked_m, int64_t E,
                                                      int64_t max_m, int64_t I, int64_t K, kbn_stream_t stream) {
    return kbn::mx::gemm1_masked_ue8m0_silu(A, sfa_packed, W13, sfb_packed, q, scale, sf_packed, masked_m, E, max_m, I, K, 0, nullptr,
                                            static_cast<cudaStream_t>(stream));
}
