/*
 * CPU oracle for the FP8 W8A8 hot path.  TEST INFRASTRUCTURE ONLY: this file is the
 * checker the CUDA kernels are compared against (and the timed CPU baseline); nothing
 * in the product library links or calls it.
 *
 * Every function restates, operation by operation, what kb-nano's reference does:
 *   kbo_quant_1x128          tasks/reference/L1/fp8_linear.py:41-64
 *                            (_quantize_fp8_per_token_group; same maths as the Triton
 *                            kernel tasks/baseline/L1/fp8_linear.py:181-215)
 *   kbo_silu_mul_quant_1x128 tasks/baseline/L1/silu_mul_quant_fp8.py:54-76
 *                            (fp32 silu -> bf16 -> *up in bf16 -> fp32 -> quant)
 *   kbo_silu_bf16_table      the silu->bf16 step alone, for all 65536 bf16 inputs
 *   kbo_block_quant_128x128  bench/kernels/scenario_registry.py:185-221
 *   kbo_gemm_nt_dequant      tasks/reference/L1/fp8_linear.py:26-38,100-104 applied to
 *                            quantised A: C = dequant(A) @ dequant(W)^T, fp32, -> bf16
 *   kbo_grouped_gemm_nt      tasks/reference/L1/moe_grouped_gemm.py:39-91,102-164
 *                            (per-row expert id, -1 rows untouched)
 *
 * Pinning: tests/test_oracle_golden.py checks these functions against fixtures generated
 * by importing the reference's own Python modules (tests/golden/make_golden.py).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define KBO_GROUP 128
#define KBO_FP8_MAX 448.0f

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = ((uint32_t)h) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even fp32 -> bf16 (NaN kept quiet), as torch's .to(bfloat16) */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* round-to-nearest-even fp32 -> float8_e4m3fn byte; caller has clamped to +-448 */
static inline uint8_t f32_to_e4m3(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint8_t)(sign | 0x7fu);          /* NaN */
    if (a >= 0x43e80000u) return (uint8_t)(sign | 0x7eu);          /* >= 464: saturate */
    if (a < 0x3c800000u) {                                         /* |x| < 2^-6: subnormal grid 2^-9 */
        float af;
        memcpy(&af, &a, 4);
        int q = (int)nearbyintf(af * 512.0f);                      /* default mode = RNE */
        return (uint8_t)(sign | (uint8_t)q);
    }
    a += 0x7ffffu + ((a >> 20) & 1u);
    uint32_t q = (a >> 20) - (120u << 3);
    if (q > 0x7eu) q = 0x7eu;
    return (uint8_t)(sign | (uint8_t)q);
}

static inline float e4m3_to_f32(uint8_t b) {
    uint32_t e = (b >> 3) & 0xfu, m = b & 7u;
    float v;
    if (e == 0) v = ldexpf((float)m, -9);
    else if (e == 15 && m == 7) v = NAN;
    else v = ldexpf(1.0f + (float)m / 8.0f, (int)e - 7);
    return (b & 0x80u) ? -v : v;
}

/* scale from the group's absmax, exactly the reference's float formula */
static inline float group_scale(float absmax, float eps, int ue8m0) {
    float a = absmax < eps ? eps : absmax;          /* clamp_min(eps) */
    float s = a / KBO_FP8_MAX;
    if (ue8m0) s = exp2f(ceilf(log2f(s)));
    return s;
}

static inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

int kbo_quant_1x128(const uint16_t* x, int64_t M, int64_t K, int64_t ldx, uint8_t* q, int64_t ldq,
                    float* scale, int64_t s_row, int64_t s_grp, float eps, int ue8m0) {
    int64_t G = (K + KBO_GROUP - 1) / KBO_GROUP;
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        for (int64_t g = 0; g < G; ++g) {
            int64_t k0 = g * KBO_GROUP, k1 = k0 + KBO_GROUP < K ? k0 + KBO_GROUP : K;
            float amax = 0.0f;
            for (int64_t k = k0; k < k1; ++k) {
                float v = fabsf(bf16_to_f32(x[m * ldx + k]));
                if (v > amax) amax = v;
            }
            float s = group_scale(amax, eps, ue8m0);
            for (int64_t k = k0; k < k1; ++k) {
                float v = bf16_to_f32(x[m * ldx + k]) / s;
                q[m * ldq + k] = f32_to_e4m3(clampf(v, -KBO_FP8_MAX, KBO_FP8_MAX));
            }
            scale[m * s_row + g * s_grp] = s;
        }
    }
    return 0;
}

static inline uint16_t silu_bf16(uint16_t gbits) {
    float g = bf16_to_f32(gbits);
    float s = g / (1.0f + expf(-g));
    return f32_to_bf16(s);
}

void kbo_silu_bf16_table(uint16_t* out) {
    for (uint32_t i = 0; i < 65536u; ++i) out[i] = silu_bf16((uint16_t)i);
}

/* in: [M, 2*N2] bf16 (gate | up); q: [M, N2]; scale element (m, g) at m*s_row + g*s_grp */
int kbo_silu_mul_quant_1x128(const uint16_t* in, int64_t M, int64_t N2, int64_t ld_in, uint8_t* q,
                             int64_t ldq, float* scale, int64_t s_row, int64_t s_grp, float eps,
                             int ue8m0) {
    int64_t G = N2 / KBO_GROUP;
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        float y[KBO_GROUP];
        for (int64_t g = 0; g < G; ++g) {
            float amax = 0.0f;
            for (int j = 0; j < KBO_GROUP; ++j) {
                uint16_t gb = in[m * ld_in + g * KBO_GROUP + j];
                uint16_t ub = in[m * ld_in + N2 + g * KBO_GROUP + j];
                float sv = bf16_to_f32(silu_bf16(gb));
                /* bf16 * bf16 evaluated in fp32 (exact) and rounded once to bf16 */
                y[j] = bf16_to_f32(f32_to_bf16(sv * bf16_to_f32(ub)));
                float a = fabsf(y[j]);
                if (a > amax) amax = a;
            }
            float s = group_scale(amax, eps, ue8m0);
            for (int j = 0; j < KBO_GROUP; ++j)
                q[m * ldq + g * KBO_GROUP + j] = f32_to_e4m3(clampf(y[j] / s, -KBO_FP8_MAX, KBO_FP8_MAX));
            scale[m * s_row + g * s_grp] = s;
        }
    }
    return 0;
}

/* w: [R, C] bf16 row-major -> q [R, C] e4m3, scale [ceil(R/128), ceil(C/128)] fp32 */
int kbo_block_quant_128x128(const uint16_t* w, int64_t R, int64_t C, uint8_t* q, float* scale,
                            float eps, int ue8m0) {
    int64_t RB = (R + 127) / 128, CB = (C + 127) / 128;
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t rb = 0; rb < RB; ++rb) {
        for (int64_t cb = 0; cb < CB; ++cb) {
            int64_t r1 = rb * 128 + 128 < R ? rb * 128 + 128 : R;
            int64_t c1 = cb * 128 + 128 < C ? cb * 128 + 128 : C;
            float amax = 0.0f;
            for (int64_t r = rb * 128; r < r1; ++r)
                for (int64_t c = cb * 128; c < c1; ++c) {
                    float v = fabsf(bf16_to_f32(w[r * C + c]));
                    if (v > amax) amax = v;
                }
            float s = group_scale(amax, eps, ue8m0);
            for (int64_t r = rb * 128; r < r1; ++r)
                for (int64_t c = cb * 128; c < c1; ++c)
                    q[r * C + c] = f32_to_e4m3(clampf(bf16_to_f32(w[r * C + c]) / s, -KBO_FP8_MAX, KBO_FP8_MAX));
            scale[rb * CB + cb] = s;
        }
    }
    return 0;
}

/* one output row: c[n] = sum_k (a[k]*sa[k/128]) * (w[n,k]*sw[n/128,k/128]) in fp32 */
static void row_gemm(const float* a_deq, const uint8_t* w, const float* sw, int64_t sw_n, int64_t sw_k,
                     int64_t N, int64_t K, const float* lut, uint16_t* c, float mul) {
    int64_t KB = (K + 127) / 128;
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t* wr = w + n * K;
        float acc = 0.0f;
        for (int64_t kb = 0; kb < KB; ++kb) {
            int64_t k1 = kb * 128 + 128 < K ? kb * 128 + 128 : K;
            float s = sw[(n / 128) * sw_n + kb * sw_k];
            float part = 0.0f;
            for (int64_t k = kb * 128; k < k1; ++k) part += a_deq[k] * (lut[wr[k]] * s);
            acc += part;
        }
        c[n] = f32_to_bf16(acc * mul);
    }
}

static void make_lut(float* lut) {
    for (int i = 0; i < 256; ++i) lut[i] = e4m3_to_f32((uint8_t)i);
}

/* A [M,K] e4m3, sa element (m,g) at m*sa_row+g*sa_grp; W [N,K] e4m3, sw (nb,kb) at nb*sw_n+kb*sw_k */
int kbo_gemm_nt_dequant(const uint8_t* A, const float* sa, int64_t sa_row, int64_t sa_grp,
                        const uint8_t* W, const float* sw, int64_t sw_n, int64_t sw_k, uint16_t* C,
                        int64_t ldc, int64_t M, int64_t N, int64_t K) {
    float lut[256];
    make_lut(lut);
#pragma omp parallel
    {
        float* a_deq = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(dynamic, 1)
        for (int64_t m = 0; m < M; ++m) {
            for (int64_t k = 0; k < K; ++k) a_deq[k] = lut[A[m * K + k]] * sa[m * sa_row + (k / 128) * sa_grp];
            row_gemm(a_deq, W, sw, sw_n, sw_k, N, K, lut, C + m * ldc, 1.0f);
        }
        free(a_deq);
    }
    return 0;
}

/* B [E,N,K], sb [E, ceil(N/128), ceil(K/128)] contiguous; row r uses expert row_expert[r] (<0: skip) */
int kbo_grouped_gemm_nt(const uint8_t* A, const float* sa, int64_t sa_row, int64_t sa_grp,
                        const uint8_t* B, const float* sb, uint16_t* C, int64_t ldc,
                        const int32_t* row_expert, int64_t M, int64_t N, int64_t K) {
    float lut[256];
    make_lut(lut);
    int64_t NB = (N + 127) / 128, KB = (K + 127) / 128;
#pragma omp parallel
    {
        float* a_deq = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(dynamic, 1)
        for (int64_t m = 0; m < M; ++m) {
            int32_t e = row_expert[m];
            if (e < 0) continue;
            for (int64_t k = 0; k < K; ++k) a_deq[k] = lut[A[m * K + k]] * sa[m * sa_row + (k / 128) * sa_grp];
            row_gemm(a_deq, B + (int64_t)e * N * K, sb + (int64_t)e * NB * KB, KB, 1, N, K, lut, C + m * ldc, 1.0f);
        }
        free(a_deq);
    }
    return 0;
}

void kbo_e4m3_decode_table(float* out256) { make_lut(out256); }
uint8_t kbo_f32_to_e4m3(float f) { return f32_to_e4m3(f); }
uint16_t kbo_f32_to_bf16(float f) { return f32_to_bf16(f); }
