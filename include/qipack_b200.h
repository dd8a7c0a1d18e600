/*
 * qipack_b200 — B200 (sm_100a) kernels for the QIPACK v6 packed linears of
 * netdur/qwen-image-cplus, behind the reference's own native operator ABI.
 *
 * Conventions (the reference's, qwen_image_cuda/src/cuda.cplus:1-60 and
 * qwen_image_cuda/cuda/gemm.cu:54-57,183-189,262-268):
 *   - every function returns a cudaError_t as int, 0 = success;
 *   - a shape or pointer the operator cannot take returns cudaErrorInvalidValue (1) before
 *     anything is launched; otherwise the launch's cudaGetLastError() is returned and
 *     asynchronous errors surface at the caller's next synchronisation;
 *   - all pointers are DEVICE pointers owned by the caller (weights are sub-ranges of one
 *     uploaded pack, so only the pack's 256-byte alignment is assumed; 16 bytes are required);
 *   - nothing is allocated and no state is kept between calls; the device used is the
 *     current one; the un-suffixed entry points launch on the legacy default stream.
 *
 * Matrix layouts (row-major):
 *   x        [m, k]     float32 or float16 activations
 *   codes    [rows, k/2] one byte per two inputs, even input in the low nibble
 *   scales   [rows, k/64] float16, one per 64-input group   (minimums likewise, W4A16 only)
 *   y        [m, n]     float32 (reference) or float16 (_ex)
 * W4A16 (scheme 5): w = code * scale + minimum, code 0..15 (int4_pack.cplus:10-11).
 * W4A4  (scheme 6): w' = code * scale, code -7..7 two's complement, weights stored rotated
 * by a block-diagonal H256; activations are rotated and quantised the same way at run time
 * (int4_pack.cplus:12-15).
 */
#ifndef QIPACK_B200_H
#define QIPACK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QI_DTYPE_F32 0
#define QI_DTYPE_F16 1

#define QI_SCHEME_W4A16 5     /* int4_pack.cplus:43 */
#define QI_SCHEME_W4A4_H256 6 /* int4_pack.cplus:44 */

/* ---- the reference's entry points, same names, arguments and error behaviour ----------- */

/* Replaces qwen_image_cuda/cuda/gemm.cu:54-57 (declared qwen_image_cuda/src/cuda.cplus:53-54).
 * x [m,k] float32 -> H256 per 256-chunk -> per 64-group scale = fp16(max(peak/7, 2^-24)),
 * code = clamp(rint(v/scale), -7, 7). k must be a multiple of 256 (the reference's kernel
 * silently assumes it; this returns 1 otherwise). Output bytes are identical to the
 * reference's for finite inputs with |x| < 2^120. */
int qi_w4a4_quantize_activations(const float *x, void *codes, void *scales, int m, int k);

/* Replaces qwen_image_cuda/cuda/gemm.cu:183-189 (cuda.cplus:55-56).
 * y[m,n] = sum over 64-groups of fma((float)int_dot, sa*sw, y). Needs m % 128 == 0,
 * n % 128 == 0, k % 256 == 0, else returns 1. */
int qi_w4a4_gemm(const void *a_codes, const void *a_scales, const void *w_codes, const void *w_scales,
                 float *y, int m, int n, int k);

/* Replaces qwen_image_cuda/cuda/gemm.cu:262-268 (cuda.cplus:57-58).
 * y = x_half . fp16(code*scale+minimum)^T, fp32 accumulate. Needs m % 128 == 0,
 * n % 128 == 0, k % 64 == 0, else returns 1. */
int qi_w4a16_gemm(const void *x_half, const void *codes, const void *scales, const void *minimums,
                  float *y, int m, int n, int k);

/* Replaces qwen_image_cuda/cuda/ops.cu:209-212 (cuda.cplus:45-46): float32 -> float16, RNE. */
int qi_f32_to_f16(const float *source, void *out, unsigned long long count);

/* ---- extended forms: stream, fp16 input/output, bias, leading dimension ----------------- */
/* `stream` is a cudaStream_t (NULL = legacy default stream). `bias` [n] float32 or NULL.
 * `y_dtype` QI_DTYPE_F32 / QI_DTYPE_F16; `ldy` = elements between rows of y (>= n; a
 * multiple of 4 for float32, 8 for float16), which lets a rank write its column slice of a
 * wider matrix. The reference's operators are these with bias NULL, float32 y, ldy = n
 * (transformer.cplus:673-713 applies no bias to packed linears). */

/* x_dtype QI_DTYPE_F32 (gemm.cu:22) or QI_DTYPE_F16 (bench/bench_w4a4.cu:33). */
int qi_w4a4_quantize_activations_ex(const void *x, int x_dtype, void *codes, void *scales, int m, int k,
                                    void *stream);

int qi_w4a4_gemm_ex(const void *a_codes, const void *a_scales, const void *w_codes, const void *w_scales,
                    const float *bias, void *y, int y_dtype, long long ldy, int m, int n, int k, void *stream);

/* Any m >= 1: rows beyond the last multiple of 128 are handled in the kernel; m <= 8 takes
 * the GEMV path below. */
int qi_w4a16_gemm_ex(const void *x_half, const void *codes, const void *scales, const void *minimums,
                     const float *bias, void *y, int y_dtype, long long ldy, int m, int n, int k, void *stream);

/* 1 <= m <= 8 activation rows (the per-block adaLN modulation linears are m = 1); n % 16 == 0,
 * k % 64 == 0. Same operator as qi_w4a16_gemm without padding m to 128. The reference has no
 * packed m = 1 path (its modulation linear is a BF16 cuBLAS call, transformer.cplus:716-730). */
int qi_w4a16_gemv_ex(const void *x_half, const void *codes, const void *scales, const void *minimums,
                     const float *bias, void *y, int y_dtype, long long ldy, int m, int n, int k, void *stream);

/* W^[n,k] = fp16(code*scale+minimum) written out as float16 [n,k] (gemm.cu:223-230): the
 * unpacked operand exactly as the GEMM kernels feed it to the tensor cores. */
int qi_w4a16_dequantize_ex(const void *codes, const void *scales, const void *minimums, void *w_half,
                           int n, int k, void *stream);

/* The exact int32 dot of every (row, column, 64-group), dots [m, n, k/64], from the same
 * kernel and tensor-core path as qi_w4a4_gemm (which also still writes y). For checking. */
int qi_w4a4_group_dots_ex(const void *a_codes, const void *a_scales, const void *w_codes, const void *w_scales,
                          float *y, int32_t *dots, int m, int n, int k, void *stream);

/* ---- the dispatcher of transformer::linear (transformer.cplus:673-713) -------------------- */

/* One packed record as the engine sees it after upload (int4_pack.cplus:76-95: scheme,
 * dimensions[0] = n, dimensions[1] = k, group_size, and the three regions as device addresses). */
typedef struct qi_packed_linear {
    uint32_t scheme;      /* QI_SCHEME_W4A16 or QI_SCHEME_W4A4_H256 */
    uint32_t group_size;  /* 64 */
    int n, k;
    const void *weights;  /* codes [n, k/2] */
    const void *scales;   /* [n, k/64] fp16 */
    const void *zeros;    /* minimums [n, k/64] fp16; NULL for scheme 6 */
    const float *bias;    /* [n] or NULL (the reference has none) */
} qi_packed_linear;

/* The activation arena of transformer.cplus:649-651: codes rows*k_max/2 bytes, code_scales
 * rows*k_max/64*2 bytes, halves rows*k_max*2 bytes. Shared by consecutive linears. */
typedef struct qi_linear_work {
    void *codes;
    void *code_scales;
    void *halves;
} qi_linear_work;

/* output[rows, n] = input[rows, k] . W^T for one record. `input` is float32 (the engine's
 * residual stream) unless input_dtype says float16. reuse_input != 0 skips quantising /
 * converting `input` because the previous linear already did so for the same input
 * (q,k,v and gate,up share one: transformer.cplus:760-762,809-810). Returns 1 for an
 * unknown scheme or group size. */
int qi_linear(const qi_packed_linear *record, const qi_linear_work *work, const void *input, int input_dtype,
              void *output, int output_dtype, long long ld_output, int rows, int reuse_input, void *stream);

/* ---- diagnostics --------------------------------------------------------------------------- */

/* Kernels of this library never spin without a bound: a wait that runs out records a code
 * (which wait, which stage) and the kernel returns. This reads and clears the code of the
 * current device (0 = healthy). Synchronises the device. */
int qi_kernel_status(unsigned int *status);

/* "qipack_b200 <version> sm_100a" */
const char *qi_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif
