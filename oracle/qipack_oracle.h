/*
 * CPU oracle for the QIPACK v6 packed-linear path (W4A16 g64 and W4A4-H256 g64).
 *
 * TEST INFRASTRUCTURE ONLY. This is a sequential restatement, in plain C, of the
 * reference's definition of the packed-linear operators; it exists so that the CUDA
 * kernels can be checked against it and so that a CPU baseline can be timed. Nothing
 * in the shipped library links, loads or calls it.
 *
 * Parity status: PINNED. The functions below are checked (tests/test_oracle.py)
 * against the known-answer tests in the reference's own unit tests
 * (qwen_image_cuda/src/int4_pack.cplus:854-938, qwen_image_cuda/src/half.cplus:81-90)
 * and against golden vectors produced by importing the reference's NumPy statement
 * of the same quantisers (tools/evaluate_int4_quantization.py) on seeded inputs
 * (tests/golden/make_golden.py, the .npz files beside it).
 *
 * Every function cites the reference file:line it follows.
 */
#ifndef QIPACK_ORACLE_H
#define QIPACK_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QIO_SCHEME_W4A16 5 /* int4_pack.cplus:43 */
#define QIO_SCHEME_W4A4_H256 6 /* int4_pack.cplus:44 */
#define QIO_GROUP 64

/* qwen_image_cuda/src/half.cplus:12-79 — software fp16 <-> fp32, round to nearest even. */
float qio_half_to_f32(uint16_t bits);
uint16_t qio_half_from_f32(float value);
float qio_half_round_f32(float value);
void qio_f32_to_f16(const float *source, uint16_t *out, size_t count); /* ops.cu:204-212 */

/* int4_pack.cplus:249-273 — radix-4 orthonormal H256 butterfly on 256 floats, in place. */
void qio_hadamard_256(float *values);

/* int4_pack.cplus:322-363 — signed codes -7..7 stored as two's complement nibbles. */
void qio_quantize_symmetric_group(const float *values, int group, int clip, uint8_t *codes,
                                  uint16_t *scale_bits);
/* int4_pack.cplus:275-320 — unsigned codes 0..15, fp16 scale and fp16 minimum. */
void qio_quantize_affine_group(const float *values, int group, int clip, uint8_t *codes,
                               uint16_t *scale_bits, uint16_t *minimum_bits);

/* int4_pack.cplus:381-425 (quantize_rows) — packs a whole fp16 matrix [n,k].
 * scheme 5: codes [n,k/2], scales [n,k/group], minimums [n,k/group].
 * scheme 6: rows rotated by H256 per 256-chunk first; minimums untouched (may be NULL).
 * Returns 0 on success, 1 on a shape the reference packer rejects. */
int qio_pack_matrix(const uint16_t *weights_f16, int n, int k, int group, int scheme, int clip,
                    uint8_t *codes, uint16_t *scales, uint16_t *minimums, int threads);

/* gemm.cu:22-52 — per row: H256 per 256-chunk, per 64-group scale = fp16(max(peak/7, 2^-24)),
 * code = clamp(rint(v/scale), -7, 7); even column in the low nibble. */
void qio_quantize_activations_f32(const float *x, int m, int k, uint8_t *codes, uint16_t *scales,
                                  int threads);
/* bench/bench_w4a4.cu:33-66 — same with fp16 input. */
void qio_quantize_activations_f16(const uint16_t *x, int m, int k, uint8_t *codes,
                                  uint16_t *scales, int threads);

/* gemm.cu:133-158 — exact int32 dot of every 64-group: dots[(row*n + col)*(k/64) + g]. */
void qio_w4a4_group_dots(const uint8_t *a_codes, const uint8_t *w_codes, int m, int n, int k,
                         int32_t *dots, int threads);
/* gemm.cu:159-168 — y += (float)dot * (sa*sw), groups ascending, fp32, fused multiply-add. */
void qio_w4a4_gemm(const uint8_t *a_codes, const uint16_t *a_scales, const uint8_t *w_codes,
                   const uint16_t *w_scales, const float *bias, float *y, int m, int n, int k,
                   int threads);
/* bench/bench_w4a4.cu:383-394 — same sum accumulated in double. */
void qio_w4a4_gemm_f64(const uint8_t *a_codes, const uint16_t *a_scales, const uint8_t *w_codes,
                       const uint16_t *w_scales, const float *bias, float *y, int m, int n, int k,
                       int threads);

/* gemm.cu:223-230 — w = fp16(fmaf(code, scale, minimum)); out [n,k] fp16 bits. */
void qio_w4a16_dequantize(const uint8_t *codes, const uint16_t *scales, const uint16_t *minimums,
                          int n, int k, uint16_t *weights_f16);
/* gemm.cu:198-260 — y = x_fp16 . dequant(W)^T. Products of two fp16 values are exact in
 * fp32; the reference accumulates them in fp32 in tensor-core order, which is unspecified,
 * so this accumulates in double and rounds once. */
void qio_w4a16_gemm(const uint16_t *x_f16, const uint8_t *codes, const uint16_t *scales,
                    const uint16_t *minimums, const float *bias, float *y, int m, int n, int k,
                    int threads);

/* Timed CPU baselines: same results within rounding, written for speed (blocked,
 * vectorisable, threaded). Used only by the bench's cpu_baseline / reference arm. */
void qio_w4a4_linear_fast(const uint16_t *x_f16, const uint8_t *w_codes, const uint16_t *w_scales,
                          float *y, int m, int n, int k, int threads);
void qio_w4a16_linear_fast(const uint16_t *x_f16, const uint8_t *codes, const uint16_t *scales,
                           const uint16_t *minimums, float *y, int m, int n, int k, int threads);

int qio_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
