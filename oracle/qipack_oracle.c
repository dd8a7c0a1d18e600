/*
 * CPU oracle for the QIPACK v6 packed-linear path. TEST INFRASTRUCTURE ONLY — see
 * qipack_oracle.h for scope and parity status (PINNED against the reference's unit-test
 * known answers and its NumPy evaluator).
 *
 * Build: make -C oracle   (gcc, -ffp-contract=off: every fused multiply-add below is an
 * explicit fmaf/fma, exactly where the reference's nvcc build contracts one).
 */
#include "qipack_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* Smallest positive fp16 value: int4_pack.cplus:53, gemm.cu:45. */
static const float SCALE_FLOOR = 5.9604645e-08f;

int qio_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* An explicit count wins over OMP_NUM_THREADS (launchers such as torch.distributed.run export
 * OMP_NUM_THREADS=1 to every rank); 0 or less means OpenMP's own default. */
static int pick_threads(int threads) {
    if (threads > 0) return threads > 1024 ? 1024 : threads;
    return qio_max_threads();
}

/* ---- fp16 (half.cplus:12-79) ---------------------------------------------------- */

static inline float bits_to_f32(uint32_t bits) {
    float value;
    memcpy(&value, &bits, 4);
    return value;
}

static inline uint32_t f32_to_bits(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    return bits;
}

/* half.cplus:12-34 */
float qio_half_to_f32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    const uint32_t exponent = ((uint32_t)h >> 10) & 0x1Fu;
    uint32_t mantissa = (uint32_t)h & 0x3FFu;
    if (exponent == 0) {
        if (mantissa == 0) return bits_to_f32(sign);
        int unbiased = -14;
        while ((mantissa & 0x400u) == 0) {
            mantissa <<= 1;
            unbiased -= 1;
        }
        mantissa &= 0x3FFu;
        return bits_to_f32(sign | ((uint32_t)(unbiased + 127) << 23) | (mantissa << 13));
    }
    if (exponent == 31) return bits_to_f32(sign | 0x7F800000u | (mantissa << 13));
    return bits_to_f32(sign | ((exponent + 127 - 15) << 23) | (mantissa << 13));
}

/* half.cplus:36-75 */
uint16_t qio_half_from_f32(float value) {
    const uint32_t bits = f32_to_bits(value);
    const uint32_t sign = (bits >> 16) & 0x8000u;
    const uint32_t exponent = (bits >> 23) & 0xFFu;
    const uint32_t mantissa = bits & 0x7FFFFFu;
    if (exponent == 0xFF) return (uint16_t)(sign | (mantissa == 0 ? 0x7C00u : 0x7E00u));
    const int half_exponent = (int)exponent - 127 + 15;
    if (half_exponent >= 31) return (uint16_t)(sign | 0x7C00u);
    if (half_exponent <= 0) {
        if (half_exponent < -10) return (uint16_t)sign;
        const uint32_t significand = mantissa | 0x800000u;
        const uint32_t shift = (uint32_t)(14 - half_exponent);
        uint32_t rounded = significand >> shift;
        const uint32_t remainder = significand & ((1u << shift) - 1u);
        const uint32_t halfway = 1u << (shift - 1);
        if (remainder > halfway || (remainder == halfway && (rounded & 1u))) rounded += 1;
        return (uint16_t)(sign | rounded);
    }
    uint32_t encoded = sign | ((uint32_t)half_exponent << 10) | (mantissa >> 13);
    const uint32_t remainder = mantissa & 0x1FFFu;
    if (remainder > 0x1000u || (remainder == 0x1000u && (encoded & 1u))) encoded += 1;
    return (uint16_t)encoded;
}

/* half.cplus:77-79 */
float qio_half_round_f32(float value) { return qio_half_to_f32(qio_half_from_f32(value)); }

/* ops.cu:204-212 */
void qio_f32_to_f16(const float *source, uint16_t *out, size_t count) {
    for (size_t i = 0; i < count; ++i) out[i] = qio_half_from_f32(source[i]);
}

/* ---- H256 (int4_pack.cplus:249-273; gemm.cu:29-39 applies the same passes) -------- */

void qio_hadamard_256(float *values) {
    for (int stride = 1; stride < 256; stride *= 4) {
        const int span = stride * 4;
        for (int base = 0; base < 256; base += span) {
            for (int offset = 0; offset < stride; ++offset) {
                const float a = values[base + offset];
                const float b = values[base + stride + offset];
                const float c = values[base + 2 * stride + offset];
                const float d = values[base + 3 * stride + offset];
                values[base + offset] = (a + b + c - d) * 0.5f;
                values[base + stride + offset] = (a + b - c + d) * 0.5f;
                values[base + 2 * stride + offset] = (a - b + c + d) * 0.5f;
                values[base + 3 * stride + offset] = (0.0f - a + b + c + d) * 0.5f;
            }
        }
    }
}

/* ---- weight quantisers ------------------------------------------------------------ */

/* int4_pack.cplus:237-247 */
static const double CLIP_CANDIDATES[7] = {1.0, 0.95, 0.9, 0.85, 0.8, 0.75, 0.7};

static inline float clampf(float value, float low, float high) {
    /* `.max(low).min(high)` in the packer, fminf(fmaxf()) in the kernels. */
    return fminf(fmaxf(value, low), high);
}

/* int4_pack.cplus:322-363 */
void qio_quantize_symmetric_group(const float *values, int group, int clip, uint8_t *codes,
                                  uint16_t *scale_bits) {
    float peak = 0.0f;
    for (int i = 0; i < group; ++i) peak = fmaxf(peak, fabsf(values[i]));
    float best_error = 0.0f;
    const int candidates = clip ? 7 : 1;
    for (int candidate = 0; candidate < candidates; ++candidate) {
        const float factor = (float)(CLIP_CANDIDATES[candidate] / 7.0);
        const float scale = qio_half_round_f32(fmaxf(peak * factor, SCALE_FLOOR));
        float error = 0.0f;
        for (int i = 0; i < group; ++i) {
            const float code = clampf(rintf(values[i] / scale), -7.0f, 7.0f);
            const float difference = code * scale - values[i];
            error = error + difference * difference;
        }
        if (candidate == 0 || error < best_error) {
            best_error = error;
            *scale_bits = qio_half_from_f32(scale);
            for (int i = 0; i < group; ++i) {
                const float code = clampf(rintf(values[i] / scale), -7.0f, 7.0f);
                codes[i] = (uint8_t)(((int32_t)code) & 15);
            }
        }
    }
}

/* int4_pack.cplus:275-320 */
void qio_quantize_affine_group(const float *values, int group, int clip, uint8_t *codes,
                               uint16_t *scale_bits, uint16_t *minimum_bits) {
    float low = values[0], high = values[0];
    for (int i = 1; i < group; ++i) {
        low = fminf(low, values[i]);
        high = fmaxf(high, values[i]);
    }
    float best_error = 0.0f;
    const int candidates = clip ? 7 : 1;
    for (int candidate = 0; candidate < candidates; ++candidate) {
        const float center = (high + low) * 0.5f;
        const float half_range = (high - low) * (float)(0.5 * CLIP_CANDIDATES[candidate]);
        const float minimum = qio_half_round_f32(center - half_range);
        const float scale =
            qio_half_round_f32(fmaxf((center + half_range - minimum) / 15.0f, SCALE_FLOOR));
        float error = 0.0f;
        for (int i = 0; i < group; ++i) {
            const float code = clampf(rintf((values[i] - minimum) / scale), 0.0f, 15.0f);
            const float difference = code * scale + minimum - values[i];
            error = error + difference * difference;
        }
        if (candidate == 0 || error < best_error) {
            best_error = error;
            *scale_bits = qio_half_from_f32(scale);
            *minimum_bits = qio_half_from_f32(minimum);
            for (int i = 0; i < group; ++i)
                codes[i] = (uint8_t)clampf(rintf((values[i] - minimum) / scale), 0.0f, 15.0f);
        }
    }
}

/* int4_pack.cplus:381-425 (quantize_rows) and :523-525 (options_valid: group in [32,256],
 * even, dividing 256) and :590-596 (W4A4 needs k % 256 == 0). */
int qio_pack_matrix(const uint16_t *weights_f16, int n, int k, int group, int scheme, int clip,
                    uint8_t *codes, uint16_t *scales, uint16_t *minimums, int threads) {
    if (group < 32 || group > 256 || (group & 1) || 256 % group != 0) return 1;
    if (n <= 0 || k <= 0 || k % group != 0) return 1;
    const int rotate = scheme == QIO_SCHEME_W4A4_H256;
    if (!rotate && scheme != QIO_SCHEME_W4A16) return 1;
    if (rotate && k % 256 != 0) return 1;
    if (!rotate && minimums == NULL) return 1;
    const int groups = k / group;
    int failed = 0;
#pragma omp parallel num_threads(pick_threads(threads))
    {
        float *row_values = (float *)malloc((size_t)k * sizeof(float));
        uint8_t group_codes[256];
        if (row_values == NULL) {
#pragma omp atomic write
            failed = 1;
        }
#pragma omp for schedule(static)
        for (int row = 0; row < n; ++row) {
            if (row_values == NULL) continue;
            for (int column = 0; column < k; ++column)
                row_values[column] = qio_half_to_f32(weights_f16[(size_t)row * k + column]);
            if (rotate)
                for (int chunk = 0; chunk < k; chunk += 256) qio_hadamard_256(row_values + chunk);
            for (int g = 0; g < groups; ++g) {
                const int start = g * group;
                uint16_t scale_bits = 0, minimum_bits = 0;
                if (rotate) {
                    qio_quantize_symmetric_group(row_values + start, group, clip, group_codes,
                                                 &scale_bits);
                } else {
                    qio_quantize_affine_group(row_values + start, group, clip, group_codes,
                                              &scale_bits, &minimum_bits);
                    minimums[(size_t)row * groups + g] = minimum_bits;
                }
                scales[(size_t)row * groups + g] = scale_bits;
                for (int pair = 0; pair < group; pair += 2)
                    codes[((size_t)row * k + start + pair) / 2] =
                        (uint8_t)(group_codes[pair] | (group_codes[pair + 1] << 4));
            }
        }
        free(row_values);
    }
    return failed;
}

/* ---- activation quantiser (gemm.cu:22-52) ---------------------------------------- */

static void quantize_row(float *row, int k, uint8_t *codes, uint16_t *scales) {
    /* gemm.cu:29-39: the butterfly runs over the whole row with i0 = (b/stride)*span + b%stride,
     * which is the same set of 4-point butterflies as one H256 per 256-chunk. */
    for (int chunk = 0; chunk < k; chunk += 256) {
        float *values = row + chunk;
        for (int stride = 1; stride < 256; stride *= 4) {
            const int span = stride * 4;
            for (int b = 0; b < 64; ++b) {
                const int i0 = (b / stride) * span + b % stride;
                const float a = values[i0], bb = values[i0 + stride], c = values[i0 + 2 * stride],
                            d = values[i0 + 3 * stride];
                values[i0] = (a + bb + c - d) * 0.5f;
                values[i0 + stride] = (a + bb - c + d) * 0.5f;
                values[i0 + 2 * stride] = (a - bb + c + d) * 0.5f;
                values[i0 + 3 * stride] = (-a + bb + c + d) * 0.5f;
            }
        }
    }
    /* gemm.cu:40-51 */
    for (int g = 0; g < k / QIO_GROUP; ++g) {
        const float *values = row + g * QIO_GROUP;
        float peak = 0.0f;
        for (int i = 0; i < QIO_GROUP; ++i) peak = fmaxf(peak, fabsf(values[i]));
        const uint16_t scale_half = qio_half_from_f32(fmaxf(peak / 7.0f, SCALE_FLOOR));
        const float scale = qio_half_to_f32(scale_half);
        for (int i = 0; i < QIO_GROUP; i += 2) {
            const int c0 = (int)clampf(rintf(values[i] / scale), -7.0f, 7.0f);
            const int c1 = (int)clampf(rintf(values[i + 1] / scale), -7.0f, 7.0f);
            codes[g * (QIO_GROUP / 2) + i / 2] = (uint8_t)((c0 & 0xF) | ((c1 & 0xF) << 4));
        }
        scales[g] = scale_half;
    }
}

void qio_quantize_activations_f32(const float *x, int m, int k, uint8_t *codes, uint16_t *scales,
                                  int threads) {
#pragma omp parallel num_threads(pick_threads(threads))
    {
        float *row = (float *)malloc((size_t)k * sizeof(float));
#pragma omp for schedule(static)
        for (int r = 0; r < m; ++r) {
            memcpy(row, x + (size_t)r * k, (size_t)k * sizeof(float));
            quantize_row(row, k, codes + (size_t)r * (k / 2), scales + (size_t)r * (k / QIO_GROUP));
        }
        free(row);
    }
}

void qio_quantize_activations_f16(const uint16_t *x, int m, int k, uint8_t *codes,
                                  uint16_t *scales, int threads) {
#pragma omp parallel num_threads(pick_threads(threads))
    {
        float *row = (float *)malloc((size_t)k * sizeof(float));
#pragma omp for schedule(static)
        for (int r = 0; r < m; ++r) {
            for (int i = 0; i < k; ++i) row[i] = qio_half_to_f32(x[(size_t)r * k + i]);
            quantize_row(row, k, codes + (size_t)r * (k / 2), scales + (size_t)r * (k / QIO_GROUP));
        }
        free(row);
    }
}

/* ---- W4A4 GEMM ---------------------------------------------------------------------- */

/* bench/bench_w4a4.cu:376-380 (nibble): even column low nibble, two's complement. */
static void unpack_signed(const uint8_t *codes, size_t count_bytes, int8_t *out) {
    for (size_t i = 0; i < count_bytes; ++i) {
        const int lo = codes[i] & 0xF, hi = codes[i] >> 4;
        out[2 * i] = (int8_t)(lo >= 8 ? lo - 16 : lo);
        out[2 * i + 1] = (int8_t)(hi >= 8 ? hi - 16 : hi);
    }
}

static inline int32_t dot64(const int8_t *a, const int8_t *b) {
    int32_t sum = 0;
    for (int i = 0; i < QIO_GROUP; ++i) sum += (int32_t)((int16_t)a[i] * (int16_t)b[i]);
    return sum;
}

void qio_w4a4_group_dots(const uint8_t *a_codes, const uint8_t *w_codes, int m, int n, int k,
                         int32_t *dots, int threads) {
    int8_t *a = (int8_t *)malloc((size_t)m * k), *w = (int8_t *)malloc((size_t)n * k);
    unpack_signed(a_codes, (size_t)m * k / 2, a);
    unpack_signed(w_codes, (size_t)n * k / 2, w);
    const int groups = k / QIO_GROUP;
#pragma omp parallel for schedule(static) num_threads(pick_threads(threads))
    for (int row = 0; row < m; ++row)
        for (int col = 0; col < n; ++col)
            for (int g = 0; g < groups; ++g)
                dots[((size_t)row * n + col) * groups + g] =
                    dot64(a + (size_t)row * k + g * QIO_GROUP, w + (size_t)col * k + g * QIO_GROUP);
    free(a);
    free(w);
}

static void w4a4_gemm_impl(const uint8_t *a_codes, const uint16_t *a_scales, const uint8_t *w_codes,
                           const uint16_t *w_scales, const float *bias, float *y, int m, int n,
                           int k, int threads, int use_double) {
    int8_t *a = (int8_t *)malloc((size_t)m * k), *w = (int8_t *)malloc((size_t)n * k);
    const int groups = k / QIO_GROUP;
    float *sa = (float *)malloc((size_t)m * groups * sizeof(float));
    float *sw = (float *)malloc((size_t)n * groups * sizeof(float));
    unpack_signed(a_codes, (size_t)m * k / 2, a);
    unpack_signed(w_codes, (size_t)n * k / 2, w);
    for (size_t i = 0; i < (size_t)m * groups; ++i) sa[i] = qio_half_to_f32(a_scales[i]);
    for (size_t i = 0; i < (size_t)n * groups; ++i) sw[i] = qio_half_to_f32(w_scales[i]);
#pragma omp parallel for schedule(static) num_threads(pick_threads(threads))
    for (int row = 0; row < m; ++row) {
        for (int col = 0; col < n; ++col) {
            if (use_double) {
                /* bench_w4a4.cu:388-393 */
                double total = 0.0;
                for (int g = 0; g < groups; ++g) {
                    const int32_t sum = dot64(a + (size_t)row * k + g * QIO_GROUP,
                                              w + (size_t)col * k + g * QIO_GROUP);
                    total += (double)sum * sa[(size_t)row * groups + g] * sw[(size_t)col * groups + g];
                }
                if (bias) total += (double)bias[col];
                y[(size_t)row * n + col] = (float)total;
            } else {
                /* gemm.cu:159-168: accumulators += (float)partial * (sa * sw), contracted
                 * by nvcc into one fused multiply-add per group, groups ascending. */
                float total = 0.0f;
                for (int g = 0; g < groups; ++g) {
                    const int32_t sum = dot64(a + (size_t)row * k + g * QIO_GROUP,
                                              w + (size_t)col * k + g * QIO_GROUP);
                    const float scale = sa[(size_t)row * groups + g] * sw[(size_t)col * groups + g];
                    total = fmaf((float)sum, scale, total);
                }
                if (bias) total = total + bias[col];
                y[(size_t)row * n + col] = total;
            }
        }
    }
    free(a);
    free(w);
    free(sa);
    free(sw);
}

void qio_w4a4_gemm(const uint8_t *a_codes, const uint16_t *a_scales, const uint8_t *w_codes,
                   const uint16_t *w_scales, const float *bias, float *y, int m, int n, int k,
                   int threads) {
    w4a4_gemm_impl(a_codes, a_scales, w_codes, w_scales, bias, y, m, n, k, threads, 0);
}

void qio_w4a4_gemm_f64(const uint8_t *a_codes, const uint16_t *a_scales, const uint8_t *w_codes,
                       const uint16_t *w_scales, const float *bias, float *y, int m, int n, int k,
                       int threads) {
    w4a4_gemm_impl(a_codes, a_scales, w_codes, w_scales, bias, y, m, n, k, threads, 1);
}

/* ---- W4A16 GEMM --------------------------------------------------------------------- */

/* gemm.cu:223-230 */
void qio_w4a16_dequantize(const uint8_t *codes, const uint16_t *scales, const uint16_t *minimums,
                          int n, int k, uint16_t *weights_f16) {
    const int groups = k / QIO_GROUP;
    for (int row = 0; row < n; ++row)
        for (int g = 0; g < groups; ++g) {
            const float scale = qio_half_to_f32(scales[(size_t)row * groups + g]);
            const float minimum = qio_half_to_f32(minimums[(size_t)row * groups + g]);
            for (int i = 0; i < QIO_GROUP; i += 2) {
                const uint8_t byte = codes[((size_t)row * k + g * QIO_GROUP + i) / 2];
                uint16_t *out = weights_f16 + (size_t)row * k + g * QIO_GROUP + i;
                out[0] = qio_half_from_f32(fmaf((float)(byte & 0x0F), scale, minimum));
                out[1] = qio_half_from_f32(fmaf((float)(byte >> 4), scale, minimum));
            }
        }
}

void qio_w4a16_gemm(const uint16_t *x_f16, const uint8_t *codes, const uint16_t *scales,
                    const uint16_t *minimums, const float *bias, float *y, int m, int n, int k,
                    int threads) {
    uint16_t *w_half = (uint16_t *)malloc((size_t)n * k * sizeof(uint16_t));
    float *w = (float *)malloc((size_t)n * k * sizeof(float));
    float *x = (float *)malloc((size_t)m * k * sizeof(float));
    qio_w4a16_dequantize(codes, scales, minimums, n, k, w_half);
    for (size_t i = 0; i < (size_t)n * k; ++i) w[i] = qio_half_to_f32(w_half[i]);
    for (size_t i = 0; i < (size_t)m * k; ++i) x[i] = qio_half_to_f32(x_f16[i]);
#pragma omp parallel for schedule(static) num_threads(pick_threads(threads))
    for (int row = 0; row < m; ++row)
        for (int col = 0; col < n; ++col) {
            const float *xr = x + (size_t)row * k, *wr = w + (size_t)col * k;
            double lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int i = 0; i < k; i += 8)
                for (int j = 0; j < 8; ++j) lanes[j] += (double)xr[i + j] * (double)wr[i + j];
            double total = ((lanes[0] + lanes[1]) + (lanes[2] + lanes[3])) +
                           ((lanes[4] + lanes[5]) + (lanes[6] + lanes[7]));
            if (bias) total += (double)bias[col];
            y[(size_t)row * n + col] = (float)total;
        }
    free(w_half);
    free(w);
    free(x);
}

/* ---- timed CPU baselines -------------------------------------------------------------
 * The reference has no CPU implementation of these linears inside its engine; its CPU
 * statement is `Mode.activations(x) @ Mode.prepare(W).T`
 * (tools/evaluate_int4_quantization.py:193-211,227-234). These two functions are that
 * operator for already-packed weights, blocked over rows so that the weights stream once
 * per 16 rows, threaded over row blocks. */

enum { ROW_BLOCK = 16 };

void qio_w4a4_linear_fast(const uint16_t *x_f16, const uint8_t *w_codes, const uint16_t *w_scales,
                          float *y, int m, int n, int k, int threads) {
    const int groups = k / QIO_GROUP;
    uint8_t *a_codes = (uint8_t *)malloc((size_t)m * k / 2);
    uint16_t *a_scales = (uint16_t *)malloc((size_t)m * groups * sizeof(uint16_t));
    qio_quantize_activations_f16(x_f16, m, k, a_codes, a_scales, threads);
    int8_t *a = (int8_t *)malloc((size_t)m * k), *w = (int8_t *)malloc((size_t)n * k);
    float *sa = (float *)malloc((size_t)m * groups * sizeof(float));
    float *sw = (float *)malloc((size_t)n * groups * sizeof(float));
    unpack_signed(a_codes, (size_t)m * k / 2, a);
    unpack_signed(w_codes, (size_t)n * k / 2, w);
    for (size_t i = 0; i < (size_t)m * groups; ++i) sa[i] = qio_half_to_f32(a_scales[i]);
    for (size_t i = 0; i < (size_t)n * groups; ++i) sw[i] = qio_half_to_f32(w_scales[i]);
#pragma omp parallel for schedule(dynamic) num_threads(pick_threads(threads))
    for (int row0 = 0; row0 < m; row0 += ROW_BLOCK) {
        const int rows = m - row0 < ROW_BLOCK ? m - row0 : ROW_BLOCK;
        for (int col = 0; col < n; ++col) {
            float totals[ROW_BLOCK];
            for (int r = 0; r < rows; ++r) totals[r] = 0.0f;
            for (int g = 0; g < groups; ++g) {
                const int8_t *wg = w + (size_t)col * k + g * QIO_GROUP;
                const float sw_g = sw[(size_t)col * groups + g];
                for (int r = 0; r < rows; ++r) {
                    const int32_t sum = dot64(a + (size_t)(row0 + r) * k + g * QIO_GROUP, wg);
                    totals[r] = fmaf((float)sum, sa[(size_t)(row0 + r) * groups + g] * sw_g, totals[r]);
                }
            }
            for (int r = 0; r < rows; ++r) y[(size_t)(row0 + r) * n + col] = totals[r];
        }
    }
    free(a_codes);
    free(a_scales);
    free(a);
    free(w);
    free(sa);
    free(sw);
}

void qio_w4a16_linear_fast(const uint16_t *x_f16, const uint8_t *codes, const uint16_t *scales,
                           const uint16_t *minimums, float *y, int m, int n, int k, int threads) {
    uint16_t *w_half = (uint16_t *)malloc((size_t)n * k * sizeof(uint16_t));
    float *w = (float *)malloc((size_t)n * k * sizeof(float));
    float *x = (float *)malloc((size_t)m * k * sizeof(float));
    qio_w4a16_dequantize(codes, scales, minimums, n, k, w_half);
#pragma omp parallel for schedule(static) num_threads(pick_threads(threads))
    for (int row = 0; row < n; ++row)
        for (int i = 0; i < k; ++i) w[(size_t)row * k + i] = qio_half_to_f32(w_half[(size_t)row * k + i]);
#pragma omp parallel for schedule(static) num_threads(pick_threads(threads))
    for (int row = 0; row < m; ++row)
        for (int i = 0; i < k; ++i) x[(size_t)row * k + i] = qio_half_to_f32(x_f16[(size_t)row * k + i]);
#pragma omp parallel for schedule(dynamic) num_threads(pick_threads(threads))
    for (int row0 = 0; row0 < m; row0 += ROW_BLOCK) {
        const int rows = m - row0 < ROW_BLOCK ? m - row0 : ROW_BLOCK;
        for (int col = 0; col < n; ++col) {
            const float *wr = w + (size_t)col * k;
            for (int r = 0; r < rows; ++r) {
                const float *xr = x + (size_t)(row0 + r) * k;
                float lanes[16];
                for (int j = 0; j < 16; ++j) lanes[j] = 0.0f;
                for (int i = 0; i < k; i += 16)
                    for (int j = 0; j < 16; ++j) lanes[j] = fmaf(xr[i + j], wr[i + j], lanes[j]);
                float total = 0.0f;
                for (int j = 0; j < 16; ++j) total += lanes[j];
                y[(size_t)(row0 + r) * n + col] = total;
            }
        }
    }
    free(w_half);
    free(w);
    free(x);
}
