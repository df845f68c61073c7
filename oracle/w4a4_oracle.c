/*
 * CPU oracle for the INT4 W4A4 linear-layer path  --  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference project
 * (rib12316/WUSH_int4_kernel).  It is a checker: only the test-suite, the
 * smoke test and the CPU-baseline leg of the benchmark may call it.  Nothing
 * in the shipped CUDA path links, imports or falls back to it.
 *
 * Parity is pinned: tests/golden/ holds vectors produced by running the
 * reference's own Python (my_int4/rtn_int4.py and the ref_fused mirror of
 * tests/test_sw2.py) in a CPU container; tests/test_oracle_golden.py checks
 * every function below against them bit for bit.
 *
 * Build: see oracle/Makefile.  -ffp-contract=off is REQUIRED: every multiply
 * and every add below must round separately, as the reference does.
 *
 * bf16 / fp16 values travel as uint16_t bit patterns.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define ORC_EXPORT __attribute__((visibility("default")))

/* 2.473650 / 7 rounded to fp32: the Gaussian-MSE clip constant for the 15-level
 * symmetric INT4 grid (reference my_int4/rtn_int4.py:19, csrc/quant_int4.cu:79). */
static const float ORC_C_CLIP = 0.35337862372398376f;

static inline float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even fp32 -> bf16, NaN kept quiet (torch .to(bfloat16)). */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* round-to-nearest-even fp32 -> fp16 (torch .to(float16)). */
static inline uint16_t f32_to_f16(float f) {
    _Float16 h = (_Float16)f;
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
}

static inline uint16_t f64_to_f16(double d) {
    _Float16 h = (_Float16)d;
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
}

static inline int nib_lo(uint8_t b) { return ((int)(b & 0xF) ^ 8) - 8; }
static inline int nib_hi(uint8_t b) { return ((int)(b >> 4) ^ 8) - 8; }

/* ---------------------------------------------------------------------------
 * One group of 32 fp32 values -> 16 packed bytes + one bf16 scale.
 * Follows my_int4/rtn_int4.py:22-55 (and its CUDA twin csrc/quant_int4.cu:63-95):
 *   s1 = sum x_i, s2 = sum (x_i * x_i), i ascending, every op rounded to fp32;
 *   mean = s1/32; var = s2/32 - mean*mean;
 *   scale = var >= 0 ? sqrt(var)*C + 1e-8 : 1.0   (NaN compares false -> 1.0);
 *   scale is stored as bf16 and the CODES use the bf16-rounded value;
 *   q = clamp(round_half_even(x / scale), -7, 7);
 *   byte i = (q[2i] & 0xF) | (q[2i+1] & 0xF) << 4.
 * ------------------------------------------------------------------------- */
static void quant_group(const float* v, uint8_t* q, uint16_t* s) {
    float s1 = 0.f, s2 = 0.f;
    for (int i = 0; i < 32; ++i) {
        s1 = s1 + v[i];
        float sq = v[i] * v[i];
        s2 = s2 + sq;
    }
    float mean = s1 / 32.0f;
    float mm = mean * mean;
    float var = s2 / 32.0f - mm;
    float scale = 1.0f;
    if (var >= 0.f) {
        float t = sqrtf(var) * ORC_C_CLIP;
        scale = t + 1e-8f;
    }
    uint16_t sb = f32_to_bf16(scale);
    *s = sb;
    scale = bf16_to_f32(sb);
    for (int i = 0; i < 32; i += 2) {
        float y0 = rintf(v[i] / scale);
        float y1 = rintf(v[i + 1] / scale);
        y0 = y0 < -7.f ? -7.f : (y0 > 7.f ? 7.f : y0);
        y1 = y1 < -7.f ? -7.f : (y1 > 7.f ? 7.f : y1);
        int q0 = (y0 == y0) ? (int)y0 : 0; /* NaN is outside the contract */
        int q1 = (y1 == y1) ? (int)y1 : 0;
        q[i / 2] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));
    }
}

/* a1: sigma-clip G=32 quantisation of bf16 input (my_int4/rtn_int4.py:33-55). */
ORC_EXPORT void orc_quant_int4(const uint16_t* x, int64_t n_groups, uint8_t* q, uint16_t* s) {
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < n_groups; ++g) {
        float v[32];
        for (int i = 0; i < 32; ++i) v[i] = bf16_to_f32(x[g * 32 + i]);
        quant_group(v, q + g * 16, s + g);
    }
}

/* Same chain from fp32 input (rtn_int4.quant_int4 accepts any float tensor; the
 * fused mirror feeds it un-rounded fp32 transform outputs, tests/test_sw2.py:24). */
ORC_EXPORT void orc_quant_int4_f32(const float* x, int64_t n_groups, uint8_t* q, uint16_t* s) {
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < n_groups; ++g) quant_group(x + g * 32, q + g * 16, s + g);
}

/* a3: serial fp32 block transform, the bit-level mirror of tests/test_sw2.py:12-23
 * (== csrc/fused_tq_int4.cu:48-58): out[r][g][j] = sum_i x[r][g][i] * T[g][j][i],
 * i ascending, product and sum rounded separately, accumulator starts at +0. */
ORC_EXPORT void orc_transform_f32(const uint16_t* x, const uint16_t* t, int64_t rows, int64_t C,
                                  float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t g = 0; g < C; ++g) {
            float xv[32];
            const uint16_t* xg = x + (r * C + g) * 32;
            const uint16_t* tg = t + g * 1024;
            for (int i = 0; i < 32; ++i) xv[i] = bf16_to_f32(xg[i]);
            for (int j = 0; j < 32; ++j) {
                float acc = 0.f;
                for (int i = 0; i < 32; ++i) {
                    float p = xv[i] * bf16_to_f32(tg[j * 32 + i]);
                    acc = acc + p;
                }
                out[(r * C + g) * 32 + j] = acc;
            }
        }
    }
}

/* a4: fused transform + quantisation, bit-exact anchor (tests/test_sw2.py:12-24,
 * csrc/fused_tq_int4.cu:27-85): transform in fp32 (not rounded to bf16), then a1. */
ORC_EXPORT void orc_fused_tq(const uint16_t* x, const uint16_t* t, int64_t rows, int64_t C,
                             uint8_t* q, uint16_t* s) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t g = 0; g < C; ++g) {
            float xv[32], xj[32];
            const uint16_t* xg = x + (r * C + g) * 32;
            const uint16_t* tg = t + g * 1024;
            for (int i = 0; i < 32; ++i) xv[i] = bf16_to_f32(xg[i]);
            for (int j = 0; j < 32; ++j) {
                float acc = 0.f;
                for (int i = 0; i < 32; ++i) {
                    float p = xv[i] * bf16_to_f32(tg[j * 32 + i]);
                    acc = acc + p;
                }
                xj[j] = acc;
            }
            quant_group(xj, q + (r * C + g) * 16, s + r * C + g);
        }
    }
}

/* a2: nibble sign-extension times scale -> fp32 (my_int4/rtn_int4.py:58-68). */
ORC_EXPORT void orc_dequant(const uint8_t* q, const uint16_t* s, int64_t rows, int64_t K,
                            float* out) {
    const int64_t G = K / 32;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t g = 0; g < G; ++g) {
            float sc = bf16_to_f32(s[r * G + g]);
            const uint8_t* qb = q + r * (K / 2) + g * 16;
            float* o = out + r * K + g * 32;
            for (int b = 0; b < 16; ++b) {
                o[2 * b] = (float)nib_lo(qb[b]) * sc;
                o[2 * b + 1] = (float)nib_hi(qb[b]) * sc;
            }
        }
}

static inline int group_dot(const uint8_t* a, const uint8_t* b) {
    int d = 0;
    for (int i = 0; i < 16; ++i) d += nib_lo(a[i]) * nib_lo(b[i]) + nib_hi(a[i]) * nib_hi(b[i]);
    return d;
}

/* Exact per-group integer partial sums P[m][n][g] = sum_{k in g} qa*qw
 * (csrc/gemm_int4.cu:11-16 states the contract; |P| <= 2048). */
ORC_EXPORT void orc_group_partials(const uint8_t* xq, const uint8_t* wq, int64_t M, int64_t N,
                                   int64_t K, int32_t* P) {
    const int64_t G = K / 32, K2 = K / 2;
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n)
            for (int64_t g = 0; g < G; ++g)
                P[(m * N + n) * G + g] = group_dot(xq + m * K2 + g * 16, wq + n * K2 + g * 16);
}

/* fp64 arbiter: Y[m][n] = sum_g sx[m][g]*sw[n][g]*P_g in double.  Equal (to fp64
 * rounding) to dequant(...).double() @ dequant(...).double().T, the arbiter of
 * tests/test_p13.py:23 and tests/test_s3.py:17-19. */
ORC_EXPORT void orc_gemm_f64(const uint8_t* xq, const uint16_t* xs, const uint8_t* wq,
                             const uint16_t* ws, int64_t M, int64_t N, int64_t K, double* y) {
    const int64_t G = K / 32, K2 = K / 2;
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            double acc = 0.0;
            for (int64_t g = 0; g < G; ++g) {
                int d = group_dot(xq + m * K2 + g * 16, wq + n * K2 + g * 16);
                acc += (double)d * (double)bf16_to_f32(xs[m * G + g]) *
                       (double)bf16_to_f32(ws[n * G + g]);
            }
            y[m * N + n] = acc;
        }
}

/* a2/a8: the reference's fp32 W4A4 product rounded to fp16
 * (my_int4/rtn_int4.py:71-75: dequantise both sides to fp32, fp32 matmul, fp16).
 * The summation order of a BLAS matmul is not part of the contract, so this uses
 * the group order of the CUDA kernels (csrc/gemm_int4.cu:60-79): exact integer dot
 * per group, acc += (float)dot * sx * sw in fp32.  It is the timed CPU baseline. */
ORC_EXPORT void orc_gemm_f16(const uint8_t* xq, const uint16_t* xs, const uint8_t* wq,
                             const uint16_t* ws, int64_t M, int64_t N, int64_t K, uint16_t* y) {
    const int64_t G = K / 32, K2 = K / 2;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t m = 0; m < M; ++m) {
            float acc = 0.f;
            for (int64_t g = 0; g < G; ++g) {
                int d = group_dot(xq + m * K2 + g * 16, wq + n * K2 + g * 16);
                float t = (float)d * bf16_to_f32(xs[m * G + g]);
                t = t * bf16_to_f32(ws[n * G + g]);
                acc = acc + t;
            }
            y[m * N + n] = f32_to_f16(acc);
        }
    }
}

/* Round an fp64 matrix to fp16 (for comparing against fp16 kernel outputs). */
ORC_EXPORT void orc_f64_to_f16(const double* in, int64_t n, uint16_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = f64_to_f16(in[i]);
}

/* Per-tensor quantisation of the reference's accuracy-free route
 * (csrc/fast_path.cu:17-39, mirrored by tests/test_p12.py:22-27):
 * q = clamp(round_half_even(x * inv_scale), -7, 7), fp32 multiply, no division. */
ORC_EXPORT void orc_quant_tensor_scale(const uint16_t* x, int64_t n, float inv_scale, uint8_t* q) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n / 2; ++i) {
        float y0 = rintf(bf16_to_f32(x[2 * i]) * inv_scale);
        float y1 = rintf(bf16_to_f32(x[2 * i + 1]) * inv_scale);
        y0 = y0 < -7.f ? -7.f : (y0 > 7.f ? 7.f : y0);
        y1 = y1 < -7.f ? -7.f : (y1 > 7.f ? 7.f : y1);
        int q0 = (y0 == y0) ? (int)y0 : 0, q1 = (y1 == y1) ? (int)y1 : 0;
        q[i] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));
    }
}

/* Per-tensor-scale GEMM (csrc/gemm_cutlass_int4.cu:39-59): full-K int32
 * accumulation, D = fp16(alpha * (float)acc). */
ORC_EXPORT void orc_gemm_tensor_scale(const uint8_t* xq, const uint8_t* wq, int64_t M, int64_t N,
                                      int64_t K, float alpha, uint16_t* y, int32_t* acc_out) {
    const int64_t K2 = K / 2;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n)
        for (int64_t m = 0; m < M; ++m) {
            int32_t acc = 0;
            const uint8_t* a = xq + m * K2;
            const uint8_t* b = wq + n * K2;
            for (int64_t i = 0; i < K2; ++i)
                acc += nib_lo(a[i]) * nib_lo(b[i]) + nib_hi(a[i]) * nib_hi(b[i]);
            if (acc_out) acc_out[m * N + n] = acc;
            if (y) y[m * N + n] = f32_to_f16(alpha * (float)acc);
        }
}

/* Whole layer as the reference times it (bench/exp_p13_official.py:31-39):
 * fused transform+quant of the activations, then the W4A4 product.  Used as the
 * CPU baseline; scratch (xq, xs) is supplied by the caller. */
ORC_EXPORT void orc_layer(const uint16_t* x, const uint16_t* t, const uint8_t* wq,
                          const uint16_t* ws, int64_t M, int64_t N, int64_t K, uint8_t* xq,
                          uint16_t* xs, uint16_t* y) {
    orc_fused_tq(x, t, M, K / 32, xq, xs);
    orc_gemm_f16(xq, xs, wq, ws, M, N, K, y);
}

ORC_EXPORT int orc_abi_version(void) { return 1; }
