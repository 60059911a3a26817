/*
 * CPU oracle for the W4A16 unpack / dequant / matmul path, plain C + OpenMP.
 *
 * TEST INFRASTRUCTURE ONLY: the checker for the CUDA kernels and the timed CPU
 * baseline of the benchmark.  The product library never links or calls it.
 *
 * Each function restates arithmetic the QuantForge reference defines
 * (paths inside the reference project):
 *   qfo_unpack_int4      lib/Transforms/LowerUnpackToArith.cpp:173-214
 *                        python/quantforge/baseline.py:34-49
 *   qfo_unpack_words     lib/Transforms/LowerUnpackToNVVM.cpp:221-280
 *   qfo_dequant          lib/Transforms/LowerDequantToArith.cpp:141-159
 *                        (zp == 0: lib/Transforms/CanonicalizeDequantZeroPoint.cpp:177-192)
 *   qfo_w4a16_linear     lib/Transforms/ConvertLinalgToQuantForge.cpp:185-203
 *                        python/quantforge/baseline.py:64-72
 * generalised to per-(group, n) scale / zero, f16 or bf16 storage and fp32
 * accumulation.  Parity of the generalisation is not pinned by any reference
 * vector; the per-channel f16 case (group == K) is pinned through the numpy
 * twin (oracle/qf_oracle.py) against outputs of the reference's own functions.
 *
 * 16-bit floats cross this interface as uint16 bit patterns.
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include <stdlib.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { QFO_F16 = 0, QFO_BF16 = 1, QFO_F32 = 2 };

static inline float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static inline float f16_to_f32(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}
static inline uint16_t f32_to_f16(float f) {
    _Float16 v = (_Float16)f; /* round-to-nearest-even */
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}
static inline float load16(const uint16_t *p, int dtype) {
    return dtype == QFO_F16 ? f16_to_f32(*p) : bf16_to_f32(*p);
}
static inline float round16(float f, int dtype) {
    if (dtype == QFO_F16) return f16_to_f32(f32_to_f16(f));
    if (dtype == QFO_BF16) return bf16_to_f32(f32_to_bf16(f));
    return f;
}

int qfo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Sets the thread count of the following calls (a launcher may have exported OMP_NUM_THREADS=1). */
void qfo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* out[r, 2i] = b & 0xF ; out[r, 2i+1] = (b >> 4) & 0xF on the raw byte. */
void qfo_unpack_int4(const uint8_t *packed, int8_t *out, int64_t rows, int64_t packed_cols) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const uint8_t *src = packed + r * packed_cols;
        int8_t *dst = out + r * packed_cols * 2;
        for (int64_t i = 0; i < packed_cols; ++i) {
            uint8_t b = src[i];
            dst[2 * i] = (int8_t)(b & 0x0F);
            dst[2 * i + 1] = (int8_t)((b >> 4) & 0x0F);
        }
    }
}

/* code[8c + i] = (w >> 4i) & 0xF */
void qfo_unpack_words(const uint32_t *words, int8_t *out, int64_t rows, int64_t words_per_row) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t c = 0; c < words_per_row; ++c) {
            uint32_t w = words[r * words_per_row + c];
            for (int i = 0; i < 8; ++i)
                out[(r * words_per_row + c) * 8 + i] = (int8_t)((w >> (4 * i)) & 0xFu);
        }
    }
}

/* zero of (group g, column n): zero_mode 0 = constant, 1 = uint4 packed 8 per uint32 along N, 2 = int8 [G,N] */
static inline int zero_at(const void *zeros, int zero_mode, int zero_const, int64_t g, int64_t n, int64_t N) {
    if (zero_mode == 0) return zero_const;
    if (zero_mode == 1) {
        const uint32_t *z = (const uint32_t *)zeros;
        return (int)((z[g * (N / 8) + n / 8] >> (4 * (n % 8))) & 0xFu);
    }
    return (int)((const int8_t *)zeros)[g * N + n];
}

/* W[n,k] = round_dtype((q - z) * s), written as float32 [N,K]. */
void qfo_dequant(const uint8_t *qweight, const uint16_t *scales, const void *zeros, int zero_mode, int zero_const,
                 float *w_out, int64_t N, int64_t K, int64_t group, int dtype) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t k = 0; k < K; ++k) {
            int64_t g = k / group;
            uint8_t b = qweight[n * (K / 2) + k / 2];
            int q = (k & 1) ? ((b >> 4) & 0xF) : (b & 0xF);
            int z = zero_at(zeros, zero_mode, zero_const, g, n, N);
            float s = load16(scales + g * N + n, dtype);
            w_out[n * K + k] = round16((float)(q - z) * s, dtype);
        }
    }
}

/*
 * Y[M,N] (float32) = X[M,K] . W^T, W dequantised on the fly row by row, fp32 accumulation.
 * The three reference passes (unpack, dequant, matmul) are fused per output row;
 * the arithmetic per element is unchanged.
 */
void qfo_w4a16_linear(const uint16_t *x, const uint8_t *qweight, const uint16_t *scales, const void *zeros,
                      int zero_mode, int zero_const, float *y, int64_t M, int64_t N, int64_t K, int64_t group,
                      int act_dtype, int out_dtype) {
    float *xf = (float *)malloc((size_t)M * K * sizeof(float));
    for (int64_t i = 0; i < M * K; ++i) xf[i] = load16(x + i, act_dtype);
#pragma omp parallel
    {
        float *wrow = (float *)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t n = 0; n < N; ++n) {
            for (int64_t g = 0; g < K / group; ++g) {
                float s = load16(scales + g * N + n, act_dtype);
                int z = zero_at(zeros, zero_mode, zero_const, g, n, N);
                const uint8_t *src = qweight + n * (K / 2) + g * (group / 2);
                float *dst = wrow + g * group;
                for (int64_t i = 0; i < group / 2; ++i) {
                    uint8_t b = src[i];
                    dst[2 * i] = round16((float)((int)(b & 0xF) - z) * s, act_dtype);
                    dst[2 * i + 1] = round16((float)((int)((b >> 4) & 0xF) - z) * s, act_dtype);
                }
            }
            for (int64_t m = 0; m < M; ++m) {
                const float *xr = xf + m * K;
                float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
                for (int64_t k = 0; k < K; k += 4) {
                    acc0 += xr[k] * wrow[k];
                    acc1 += xr[k + 1] * wrow[k + 1];
                    acc2 += xr[k + 2] * wrow[k + 2];
                    acc3 += xr[k + 3] * wrow[k + 3];
                }
                y[m * N + n] = round16((acc0 + acc1) + (acc2 + acc3), out_dtype);
            }
        }
        free(wrow);
    }
    free(xf);
}
