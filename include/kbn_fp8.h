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
 * called by Fp8Linear.forward (tasks/baseline/L1/fp8_linear.py:91-110,443-445). */
int kbn_fp8_gemm_nt(const void* A, const float* sa, int64_t sa_row, int64_t sa_grp, const void* B,
                    const float* sb, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                    kbn_stream_t stream);

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

/* Device status word of the GEMM kernels' bounded waits: 0 = no wait ever ran out in this
 * process.  Host pointer out; synchronises `stream` first. */
int kbn_gemm_status(int32_t* host_out, kbn_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* KBN_FP8_H */
