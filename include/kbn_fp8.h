/*
 * kbn_fp8 -- C ABI of the B200 (sm_100a) FP8 W8A8 hot path for kb-nano.
 *
 * Plain pointers and sizes only; every pointer is a device pointer unless said otherwise.
 * Every function returns 0 on success or a negative KBN_ERR_* code, never throws and never
 * synchronises the device; kernels are enqueued on `stream` (a cudaStream_t passed as void*).
 * After a non-zero return kbn_last_error() gives a message for the calling thread.
 * Strides are in ELEMENTS of the pointed-to type.  bf16 = 2-byte bfloat16, fp8 = 1-byte
 * float8_e4m3fn.  "Group" = 128 consecutive elements of the last dimension.
 *
 * Each entry point names the kb-nano interface it stands behind (paths relative to the
 * kb-nano tree).
 */
#ifndef KBN_FP8_H
#define KBN_FP8_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KBN_OK 0
#define KBN_ERR_ARG (-1)          /* bad shape / stride / alignment / null pointer */
#define KBN_ERR_CUDA (-2)         /* a CUDA runtime or driver call failed */
#define KBN_ERR_UNSUPPORTED (-3)  /* device is not sm_100, or size beyond a stated limit */
#define KBN_ERR_TIMEOUT (-4)      /* a bounded device-side wait ran out (see kbn_*_status) */

typedef void* kbn_stream_t;

int kbn_version(void);
const char* kbn_last_error(void);

/* Number of kernels this library has launched from the calling process (all threads). */
int64_t kbn_launch_count(void);

/*
 * Per-token-group activation quantisation, 1x128 groups along K.
 * Stands behind torch.ops.kb_nano_fp8.per_token_group_quant_fp8 / PerTokenGroupQuantFp8.forward
 * (tasks/baseline/L1/fp8_linear.py:157-160,234-297; Triton kernel :181-215).
 *   x      [M,K] bf16, row stride ld_x      q [M,K] fp8, row stride ld_q
 *   scale  fp32, element (m,g) at scale[m*s_row + g*s_grp]   (row-major: (G,1); column-major: (1,M))
 *   ue8m0 != 0: scale = 2^ceil(log2(max(absmax,eps)/448));  ue8m0 == 0: scale = max(absmax,eps)/448
 * K need not be a multiple of 128: a short last group is quantised over the elements it has.
 */
int kbn_quant_1x128(const void* x, int64_t M, int64_t K, int64_t ld_x, void* q, int64_t ld_q,
                    float* scale, int64_t s_row, int64_t s_grp, float eps, int ue8m0,
                    kbn_stream_t stream);
/* The same with UE8M0 scales, and sf_packed (kbn_packed_sf_rows_bytes(M, K) bytes, 16-byte aligned) also receives
 * the scales in the packed form the *_ue8m0 GEMMs read, so that a linear layer is two launches (this and the GEMM).
 * Needs K, ld_x and ld_q to be multiples of 8 and x 16-byte aligned.  Words of rows past M in the last 128-row
 * block are left unwritten (the GEMM never stores those rows). */
int kbn_quant_1x128_sf(const void* x, int64_t M, int64_t K, int64_t ld_x, void* q, int64_t ld_q,
                       float* scale, int64_t s_row, int64_t s_grp, float eps, void* sf_packed,
                       kbn_stream_t stream);

/*
 * Fused SiLU(gate)*up + 1x128 quantisation.
 * Stands behind SiluMulQuantFp8.forward (tasks/baseline/L1/silu_mul_quant_fp8.py:23-76,87-143).
 *   in  [M, 2*N2] bf16 (gate | up halves of each row), row stride ld_in;  N2 % 128 == 0
 *   q   [M, N2] fp8, row stride ld_q;  scale element (m,g) at scale[m*s_row + g*s_grp]
 * Arithmetic: s = bf16(g/(1+exp(-g))) with g widened to fp32; y = bf16(s*up); then as above on y.
 * The first call on a device also enqueues (on `stream`) a one-off kernel that fills a 128 KB
 * device-resident lookup table used for the exactly-rounded slow path.
 */
int kbn_silu_mul_quant_1x128(const void* in, int64_t M, int64_t N2, int64_t ld_in, void* q,
                             int64_t ld_q, float* scale, int64_t s_row, int64_t s_grp, float eps,
                             int ue8m0, kbn_stream_t stream);

/* Same kernel restricted to the rows that hold data, for the two grouped-GEMM layouts (the rows it
 * skips are neither read nor written):
 *   _rows:   expert-contiguous layout, row m is processed iff row_expert[m] >= 0;
 *   _list:   only the rows named in row_list[0..n_list) (entries < 0 skipped); each listed row is read and
 *            written at its own index.  The MoE layer passes the destination rows of its (token, slot) pairs,
 *            which spreads the work evenly however the rows are grouped;
 *   _masked: in [E, max_m, 2*N2] -> q [E, max_m, N2], row-major scales [E, max_m, N2/128], UE8M0,
 *            eps 1e-10; row (e, m) is processed iff m < masked_m[e].
 *   sf_packed (_list; may be null, needs ue8m0): also receives the scales of the listed rows in the packed
 *            form of the *_ue8m0 GEMMs, kbn_packed_sf_rows_bytes(rows of q, N2) bytes, rows indexed as in q.
 * kb-nano runs its kernel over every row of the padded buffer (tasks/baseline/L2/fused_experts.py:269-274). */
int kbn_silu_mul_quant_1x128_rows(const void* in, int64_t M, int64_t N2, int64_t ld_in, void* q,
                                  int64_t ld_q, float* scale, int64_t s_row, int64_t s_grp, float eps,
                                  int ue8m0, const int32_t* row_expert, kbn_stream_t stream);
int kbn_silu_mul_quant_1x128_list(const void* in, int64_t N2, int64_t ld_in, void* q, int64_t ld_q,
                                  float* scale, int64_t s_row, int64_t s_grp, float eps, int ue8m0,
                                  const int32_t* row_list, int64_t n_list, void* sf_packed,
                                  kbn_stream_t stream);
int kbn_silu_mul_quant_1x128_masked(const void* in, int64_t E, int64_t max_m, int64_t N2, void* q,
                                    float* scale, const int32_t* masked_m, kbn_stream_t stream);

/*
 * Fused RMSNorm + 1x128 quantisation, and its residual-add form: the producer of the activations the FP8
 * linears consume.  Stand behind torch.ops.kb_nano_norm.rmsnorm_fp8_quant / fused_add_rmsnorm_fp8_quant
 * (tasks/baseline/L1/rmsnorm_quant.py:25-57,63-132; kernels tasks/baseline/L1/csrc/rmsnorm_quant.cu:22-97,125-204).
 *   x [M,H] bf16, weight [H] bf16; q [M,H] fp8; scale element (m,g) at scale[m*s_row + g*s_grp], UE8M0,
 *   absmax clamp 1e-10.  H % 8 == 0, H <= 16384.
 *   add form: residual <- bf16(residual + x) (fp32 sum), the norm is taken of that rounded row, and
 *   x <- bf16(normalised row); both are modified in place like the reference.
 * Floating-point kernel: results match the reference's arithmetic up to the summation order of the
 * squares (tolerance: the harness's FP8 pair rule, bench/kernels/runner.py:265-291).
 */
int kbn_rmsnorm_quant_1x128(const void* x, const void* weight, int64_t M, int64_t H, int64_t ld_x,
                            void* q, int64_t ld_q, float* scale, int64_t s_row, int64_t s_grp,
                            float eps, kbn_stream_t stream);
int kbn_add_rmsnorm_quant_1x128(void* x, void* residual, const void* weight, int64_t M, int64_t H,
                                int64_t ld_x, int64_t ld_res, void* q, int64_t ld_q, float* scale,
                                int64_t s_row, int64_t s_grp, float eps, kbn_stream_t stream);

/* silu(gate)->bf16 for all 65536 gate bit patterns, as the kernel above computes it
 * (out: 65536 x uint16 on the device).  Used by the exhaustive parity test. */
int kbn_silu_bf16_table(void* out_u16, kbn_stream_t stream);

/*
 * Block-scaled FP8 GEMMs, "NT" form: C[m,n] = sum_kb sa[m,kb] * sb[n/128,kb] * <A[m,kb], B[n,kb]>,
 * fp32 accumulation (tcgen05 MMA, TMEM accumulators, per-128-K-block promotion), bf16 output.
 * A, B are fp8 with K contiguous (row strides K); K % 16 == 0, N % 8 == 0; all base pointers
 * 16-byte aligned.  Activation scales sa: element (m,kb) at sa[m*sa_row + kb*sa_grp].
 * Weight scales sb: fp32 [.., ceil(N/128), ceil(K/128)] contiguous (any positive value, not
 * only powers of two).
 */

/* Dense linear.  Stands behind torch.ops.kb_nano_fp8.fp8_gemm_nt, i.e. deep_gemm.fp8_gemm_nt as
 * called by Fp8Linear.forward (tasks/baseline/L1/fp8_linear.py:91-110,443-447).  bias: bf16 [N] or
 * null; it is added to the fp32 accumulator before the one rounding to bf16, as the reference's
 * F.linear(x, w, bias) does (tasks/reference/L1/fp8_linear.py:103), so the layer needs no separate
 * `output + bias` pass over [M, N]. */
int kbn_fp8_gemm_nt(const void* A, const float* sa, int64_t sa_row, int64_t sa_grp, const void* B,
                    const float* sb, const void* bias, void* C, int64_t ldc, int64_t M, int64_t N,
                    int64_t K, kbn_stream_t stream);

/* Grouped, expert-contiguous rows.  Stands behind m_grouped_fp8_gemm_nt_contiguous
 * (tasks/baseline/L1/moe_grouped_gemm.py:71-83; tasks/baseline/L1/fp8_grouped_gemm_contiguous.py:102-118).
 *   A [M_sum,K], B [E,N,K], sb [E,ceil(N/128),ceil(K/128)], C [M_sum,N],
 *   row_expert int32 [M_sum]: expert of each row, <0 = padding (row not written).
 * Each 128-row block takes its expert from its first row, so segments must be 128-aligned. */
int kbn_fp8_grouped_gemm_contig(const void* A, const float* sa, int64_t sa_row, int64_t sa_grp,
                                const void* B, const float* sb, void* C, int64_t ldc,
                                const int32_t* row_expert, int64_t M_sum, int64_t N, int64_t K,
                                int64_t E, kbn_stream_t stream);

/* Grouped, masked layout (decode / expert-parallel): A [E,max_m,K], sa element (e,m,kb) at
 * sa[e*sa_exp + m*sa_row + kb*sa_grp], B [E,N,K], C [E,max_m,N]; only rows m < masked_m[e] are
 * computed and written.  No call site in kb-nano; the layout is the one DeepGEMM's masked
 * grouped GEMM uses. */
int kbn_fp8_grouped_gemm_masked(const void* A, const float* sa, int64_t sa_exp, int64_t sa_row,
                                int64_t sa_grp, const void* B, const float* sb, void* C,
                                const int32_t* masked_m, int64_t E, int64_t max_m, int64_t N,
                                int64_t K, kbn_stream_t stream);

/*
 * UE8M0 fast path of the three GEMMs above, for scales that are all powers of two (what kb-nano's
 * activation quantisation always produces, and its weights after the UE8M0 re-quantisation of
 * tasks/baseline/L1/fp8_linear.py:492-499).  Same arithmetic contract and the same kb-nano call
 * sites as the fp32-scale entry points; the scales are passed in the packed form the block-scaled
 * tensor-core instruction reads (tcgen05.mma.kind::mxf8f6f4.block_scale), which is also the role of
 * DeepGEMM's transform_sf_into_required_layout (tasks/baseline/L1/fp8_linear.py:502-510).
 *   kbn_pack_sf_rows:    fp32 [rows, ceil(K/128)] (element (r,kb) at scale[r*s_row + kb*s_grp]) ->
 *                        kbn_packed_sf_rows_bytes(rows, K) bytes.  For the masked layout pass
 *                        rows = E*max_m (max_m % 128 == 0).
 *   kbn_pack_sf_weights: fp32 [E, ceil(N/128), ceil(K/128)] -> kbn_packed_sf_weights_bytes(E, N, K) bytes.
 *   kbn_count_non_pow2_scales: adds to *device_count the number of scales that are not positive
 *                        powers of two; a caller uses it once per weight tensor to choose the path.
 * Requirements beyond the fp32-scale kernels: contiguous-layout segments and max_m are multiples of
 * 128 rows; all pointers 16-byte aligned.
 */
int64_t kbn_packed_sf_rows_bytes(int64_t rows, int64_t K);
int64_t kbn_packed_sf_weights_bytes(int64_t E, int64_t N, int64_t K);
int kbn_pack_sf_rows(const float* scale, int64_t rows, int64_t K, int64_t s_row, int64_t s_grp,
                     void* packed, kbn_stream_t stream);
int kbn_pack_sf_weights(const float* sb, int64_t E, int64_t N, int64_t K, void* packed,
                        kbn_stream_t stream);
int kbn_count_non_pow2_scales(const float* s, int64_t n, int32_t* device_count, kbn_stream_t stream);
int kbn_fp8_gemm_nt_ue8m0(const void* A, const void* sfa_packed, const void* B,
                          const void* sfb_packed, const void* bias, void* C, int64_t ldc, int64_t M,
                          int64_t N, int64_t K, kbn_stream_t stream);
int kbn_fp8_grouped_gemm_contig_ue8m0(const void* A, const void* sfa_packed, const void* B,
                                      const void* sfb_packed, void* C, int64_t ldc,
                                      const int32_t* row_expert, int64_t M_sum, int64_t N, int64_t K,
                                      int64_t E, kbn_stream_t stream);
int kbn_fp8_grouped_gemm_masked_ue8m0(const void* A, const void* sfa_packed, const void* B,
                                      const void* sfb_packed, void* C, const int32_t* masked_m,
                                      int64_t E, int64_t max_m, int64_t N, int64_t K,
                                      kbn_stream_t stream);

/* Grouped GEMM1 of the MoE expert MLP with the activation applied in its epilogue (UE8M0 path):
 * W13 is [E, 2*I, K] with an expert's I gate rows followed by its I up rows
 * (tasks/baseline/L2/fused_experts.py:263-274 runs m_grouped_fp8_gemm_nt_contiguous, stores bf16
 * [M, 2*I] and then SiluMulQuantFp8); sfb_packed is kbn_pack_sf_weights of its [E, 2*I/128, K/128] scales.
 * Output: q e4m3 [rows, I] (row stride ld_q), scale fp32 with element strides (s_row, s_grp), and, when
 * sf_packed is not null, the same scales in the packed form (kbn_packed_sf_rows_bytes(rows, I) bytes) that
 * GEMM2 reads.  Bit-identical to kbn_fp8_grouped_gemm_*_ue8m0 into a bf16 buffer followed by
 * kbn_silu_mul_quant_1x128 (ue8m0, eps 1e-10) on it; rows that hold no data are not written.
 * I must be a multiple of 128.  The masked form writes q [E, max_m, I] and row-major scales [E, max_m, I/128]. */
int kbn_fp8_grouped_gemm_contig_ue8m0_silu(const void* A, const void* sfa_packed, const void* W13,
                                           const void* sfb_packed, void* q, int64_t ld_q, float* scale,
                                           int64_t s_row, int64_t s_grp, void* sf_packed,
                                           const int32_t* row_expert, int64_t M_sum, int64_t I, int64_t K,
                                           int64_t E, kbn_stream_t stream);
int kbn_fp8_grouped_gemm_masked_ue8m0_silu(const void* A, const void* sfa_packed, const void* W13,
                                           const void* sfb_packed, void* q, float* scale, void* sf_packed,
                                           const int32_t* masked_m, int64_t E, int64_t max_m, int64_t I,
                                           int64_t K, kbn_stream_t stream);

/*
 * Load-time re-quantisation of block-scaled FP8 weights to power-of-two scales, in place:
 * per 128x128 block  w = fp32(w_fp8) * scale,  scale <- 2^ceil(log2(max(max|w|, eps) / 448)),
 * w_fp8 <- e4m3(w / scale).  w_fp8 [E,N,K] (E = 1 for a dense weight), scale fp32 [E, ceil(N/128), ceil(K/128)].
 * Stands behind the dequantise -> deep_gemm.per_block_cast_to_fp8(use_ue8m0=True) step of
 * postprocess_fp8_weights / postprocess_fp8_weights_batched (tasks/baseline/L1/fp8_linear.py:453-554);
 * DeepGEMM (v2.1.1.post3, not in the kb-nano tree) clamps the block maximum at 1e-4: pass that as eps
 * to follow it.  After this call kbn_pack_sf_weights gives the layout the UE8M0 GEMMs read.
 */
int kbn_requant_weights_ue8m0(void* w_fp8, float* scale, int64_t E, int64_t N, int64_t K, float eps,
                              kbn_stream_t stream);

/* Device status word of the GEMM kernels' bounded waits: 0 = no wait ever ran out in this
 * process.  Host pointer out; synchronises `stream` first. */
int kbn_gemm_status(int32_t* host_out, kbn_stream_t stream);
/* Sets the word back to 0 (stream-ordered), so that one expired wait does not mark every later check. */
int kbn_gemm_clear_status(kbn_stream_t stream);

/*
 * Token permutation around the two grouped GEMMs of the FP8 MoE expert pipeline.  Together they
 * stand behind _deepgemm_permute / _deepgemm_unpermute_and_reduce
 * (tasks/baseline/L2/fused_experts.py:42-116,119-136).
 *
 * kbn_moe_aligned_rows: row capacity of the expert-contiguous buffers,
 *   round_up(T*topk + E*127, 128)  (_compute_aligned_M, tasks/baseline/L2/fused_experts.py:32-39).
 * kbn_moe_permute: a_q [T,K] fp8 + a_s [T,K/128] fp32 (row-major) + topk_ids [T,topk] int32 ->
 *   a_perm [M_cap,K], a_s_perm [M_cap,K/128]: rows grouped by expert, each expert's segment
 *     starting on a multiple of 128 rows, pairs kept in (token, slot) order inside a segment;
 *     padding rows are left unwritten;
 *   row_expert int32 [M_cap]: expert of each row, -1 for padding;
 *   dest_row int32 [T,topk]: row each (token, slot) went to (-1 if its expert id is out of range).
 *   workspace: kbn_moe_permute_workspace_bytes(T, topk, E) bytes of device scratch.
 * kbn_moe_permute_sf: the same, and a_sf_packed (kbn_packed_sf_rows_bytes(M_cap, K) bytes; may be null)
 *   also receives the moved rows' scales in the packed form of the *_ue8m0 GEMMs (scales must be powers
 *   of two); words of padding rows are left unwritten.
 * kbn_moe_unpermute_combine: out[t,:] = sum_s topk_w[t,s] * rows[dest_row[t,s],:], fp32
 *   accumulation in slot order, bf16 [T,H] out; rows is bf16 with row stride ld_rows.
 */
int64_t kbn_moe_aligned_rows(int64_t T, int64_t topk, int64_t E);
/* Front end of the sorted-token layout of kb-nano's Triton MoE path (MoeGroupedGemm.forward,
 * tasks/baseline/L1/moe_grouped_gemm.py:294-382; the lists come from moe_align_block_size): pair_expert int32
 * [n_pairs] = expert of every (token, slot) pair t, read out of sorted_ids int32 [n_sorted] (position i lies in block
 * i / block_m; entries >= n_pairs are padding) and expert_ids int32 [n_blocks]; -1 for pairs in no block.
 * sorted_ids == NULL: block i holds the single pair i.  The result is the topk_ids argument of kbn_moe_permute. */
int kbn_moe_pair_experts(const int32_t* sorted_ids, int64_t n_sorted, const int32_t* expert_ids,
                         int64_t n_blocks, int64_t block_m, int64_t n_pairs, int32_t* pair_expert,
                         kbn_stream_t stream);
int64_t kbn_moe_permute_workspace_bytes(int64_t T, int64_t topk, int64_t E);
int kbn_moe_permute(const void* a_q, const float* a_s, const int32_t* topk_ids, int64_t T,
                    int64_t topk, int64_t K, int64_t E, void* a_perm, float* a_s_perm,
                    int32_t* row_expert, int32_t* dest_row, int64_t M_cap, void* workspace,
                    int64_t workspace_bytes, kbn_stream_t stream);
int kbn_moe_permute_sf(const void* a_q, const float* a_s, const int32_t* topk_ids, int64_t T,
                       int64_t topk, int64_t K, int64_t E, void* a_perm, float* a_s_perm,
                       int32_t* row_expert, int32_t* dest_row, int64_t M_cap, void* workspace,
                       int64_t workspace_bytes, void* a_sf_packed, kbn_stream_t stream);
/* kbn_moe_permute for callers that cannot allocate device memory (a plug-in that only receives its
 * input and output tensors, a host that has frozen its memory map): identical outputs, the scratch is
 * a ~264 KB device array built into the library.  No counterpart in kb-nano.  Limits: T*topk <= 65536
 * and E <= 1024 (KBN_ERR_UNSUPPORTED beyond).  Allocates nothing; the first call on a device resolves
 * the array's address and should come before any stream capture; calls that overlap on one GPU race
 * on the shared scratch. */
int kbn_moe_permute_static(const void* a_q, const float* a_s, const int32_t* topk_ids, int64_t T,
                           int64_t topk, int64_t K, int64_t E, void* a_perm, float* a_s_perm,
                           int32_t* row_expert, int32_t* dest_row, int64_t M_cap, kbn_stream_t stream);
int kbn_moe_unpermute_combine(const void* rows, int64_t ld_rows, const int32_t* dest_row,
                              const float* topk_w, int64_t T, int64_t topk, int64_t H, void* out,
                              kbn_stream_t stream);

/*
 * Expert routing in front of the MoE pipeline, one kernel per token batch: stands behind TopKSoftmax
 * (tasks/baseline/L1/topk_softmax.py:37-60) and GroupedTopK (tasks/baseline/L1/grouped_topk.py:75-174).
 *   logits [T, E] fp32 or bf16 (logits_bf16), row stride ld; E <= 1024, topk <= 32;
 *   softmax != 0: scores = softmax(logits), else sigmoid(logits); fp32 arithmetic, or, with round_bf16,
 *     rounded to bf16 step by step (GroupedTopK scores in the logits' dtype);
 *   bias (may be null) fp32 [E]: added to the scores for the selection only (e_score_correction_bias);
 *   n_group / topk_group: the experts form n_group contiguous groups (n_group divides E, <= 32); only the
 *     topk_group groups with the best score (sum of their two largest biased scores, or their largest score
 *     without a bias) take part; n_group = topk_group = 1 switches this off;
 *   out_w fp32 [T, topk]: unbiased scores of the chosen experts, divided by max(their sum, renorm_floor) when
 *     renormalize != 0, times scale; out_ids int32 [T, topk]; both in descending order of the selection value,
 *     ties to the lower expert id.
 */
int kbn_moe_route_topk(const void* logits, int logits_bf16, int64_t ld, int64_t T, int64_t E, int softmax,
                       const float* bias, int64_t n_group, int64_t topk_group, int64_t topk,
                       int renormalize, float renorm_floor, float scale, int round_bf16, float* out_w,
                       int32_t* out_ids, kbn_stream_t stream);

/*
 * Expert-parallel FP8 MoE layer over the GPUs of one NVLink/NVSwitch box, one process per GPU.
 * Experts are split in contiguous blocks (rank r owns experts [r*E/R, (r+1)*E/R)); tokens stay on
 * their source rank.  Dispatch and combine are peer stores over NVLink issued by this library's
 * kernels; arrival is signalled with release/acquire flags whose waits are bounded (about 1 s).
 * It takes the place of the tensor-parallel all-reduce that ends kb-nano's MoE layers
 * (tasks/baseline/L1/allreduce.py:37-48 called from tasks/baseline/L2/deepseek_moe.py:301-302,
 * qwen3_moe.py:185-186, mixtral_moe.py:80-81); kb-nano has no expert-parallel path of its own.
 *
 * Bootstrap (not the hot path; allocates with cudaMalloc and maps peers with CUDA IPC):
 *   kbn_ep_create on every rank (its GPU current) -> kbn_ep_ipc_handle -> exchange the 64-byte
 *   handles by any host channel -> kbn_ep_attach(all handles, rank order).  world == 1 needs no attach.
 *   An all-zero handle maps that rank onto the caller's own buffer: a rank that never runs, whose
 *   signals never arrive (the bounded waits for it end with status 20 after about a second each).
 * kbn_ep_moe_forward: x bf16 [T,H] local tokens, topk_ids int32 [T,topk] GLOBAL expert ids,
 *   topk_w fp32 [T,topk]; w13 fp8 [E/R,2I,H] + w13_s fp32 [E/R,2I/128,H/128], w2 fp8 [E/R,H,I] +
 *   w2_s [E/R,H/128,I/128] of the LOCAL experts; out bf16 [T,H].  When both w13_sf_packed and
 *   w2_sf_packed (kbn_pack_sf_weights of the same scales) are given and max_m % 128 == 0, the expert
 *   GEMMs take the UE8M0 fast path and the fp32 scale pointers may be null.  Every rank must call it
 *   the same number of times (also with T == 0).  An expert can take at most max_m rows per call.
 * kbn_ep_moe_forward_routed: the same layer call from the router's logits instead of its choice: logits
 *   [T, E] (fp32 or bf16, row stride ld) go through the routing of kbn_moe_route_topk (same arguments, same
 *   arithmetic: tasks/baseline/L1/topk_softmax.py:37-60, tasks/baseline/L1/grouped_topk.py:75-174) inside the
 *   dispatch kernel -- one warp of the token's CTA routes while the others quantise the row -- so the layer
 *   stays at four launches with the router included.  topk is the context's.  kbn_ep_last_routing copies the
 *   weights fp32 [T, topk] and expert ids int32 [T, topk] that call chose (device to device, stream-ordered).
 * kbn_ep_status: 4 int32 {code, phase, peer, detail}; code 0 = ok, 10 = an expert overflowed max_m
 *   rows (detail = expert), 11 = expert id out of range, 20 = a wait on peer `peer` ran out in
 *   phase 1 (dispatch) or 2 (combine).  Synchronises `stream`.  The first code of a context sticks
 *   until kbn_ep_clear_status (stream-ordered) sets the four words back to 0.
 * kbn_ep_expert_phase: measurement aid.  Runs the two expert GEMMs of the UE8M0 path once more, exactly as a
 *   layer call launches them (GEMM1 with the activation epilogue, GEMM2 with the combine epilogue started
 *   while GEMM1 still runs), on the rows the last kbn_ep_moe_forward left in the receive buffers, with
 *   rows_per_expert int32 [E/R] (device) as the row counts; it exchanges no flags and leaves the step
 *   counter alone, so a caller can bracket it with events.  Every rank may call it at the same time; the
 *   result rows it re-sends are the ones the last step already delivered.
 */
typedef struct kbn_ep_ctx kbn_ep_ctx;
int kbn_ep_create(int rank, int world, int64_t experts_total, int64_t max_m, int64_t hidden,
                  int64_t inter, int64_t max_tokens, int64_t topk, kbn_ep_ctx** out);
int kbn_ep_ipc_handle(kbn_ep_ctx* ctx, void* out64);
int kbn_ep_attach(kbn_ep_ctx* ctx, const void* handles);
int64_t kbn_ep_symmetric_bytes(kbn_ep_ctx* ctx);
int kbn_ep_moe_forward(kbn_ep_ctx* ctx, const void* x_bf16, const int32_t* topk_ids,
                       const float* topk_w, int64_t T, const void* w13, const float* w13_s,
                       const void* w2, const float* w2_s, const void* w13_sf_packed,
                       const void* w2_sf_packed, void* out_bf16, kbn_stream_t stream);
int kbn_ep_moe_forward_routed(kbn_ep_ctx* ctx, const void* x_bf16, const void* logits, int logits_bf16,
                              int64_t ld, int64_t T, int softmax, const float* bias, int64_t n_group,
                              int64_t topk_group, int renormalize, float renorm_floor, float scale,
                              int round_bf16, const void* w13, const float* w13_s, const void* w2,
                              const float* w2_s, const void* w13_sf_packed, const void* w2_sf_packed,
                              void* out_bf16, kbn_stream_t stream);
int kbn_ep_last_routing(kbn_ep_ctx* ctx, float* out_w, int32_t* out_ids, int64_t T, kbn_stream_t stream);
int kbn_ep_status(kbn_ep_ctx* ctx, int32_t* host_out4, kbn_stream_t stream);
int kbn_ep_clear_status(kbn_ep_ctx* ctx, kbn_stream_t stream);
int kbn_ep_expert_phase(kbn_ep_ctx* ctx, const void* w13, const void* w13_sf_packed, const void* w2,
                        const void* w2_sf_packed, const int32_t* rows_per_expert, int64_t expected_m,
                        kbn_stream_t stream);
int kbn_ep_destroy(kbn_ep_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* KBN_FP8_H */
