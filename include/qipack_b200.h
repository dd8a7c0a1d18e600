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
 *   - the operators keep no state between calls beyond per-device facts looked up once (SM
 *     count, the kernels' shared-memory opt-in; safe from several host threads) and allocate
 *     nothing, with one exception: the W4A4 GEMM on nibble-packed operands (qi_w4a4_gemm,
 *     qi_w4a4_gemm_ex, and qi_linear on a scheme-6 record without byte-wide weights) takes
 *     (m + n) * k bytes of scratch per call from a memory pool of the library's own when it
 *     chooses its widened path (see qi_w4a4_gemm_path_ex; qi_w4a4_gemm_noalloc_ex is the form
 *     that takes none). The device used is the current one; the un-suffixed entry points launch
 *     on the legacy default stream. (The sharding context further down owns a communicator,
 *     streams and events: those are created by qi_shard_create and freed by qi_shard_destroy.)
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

/* qi_w4a4_gemm_ex on its widened path (path 2 below) without taking memory from anywhere: the widened operands go
 * into a fixed array of QI_NOALLOC_SCRATCH_BYTES that is part of the library's device code, one instance per device.
 * For callers that may not allocate while they run: a process whose device memory is handed out completely at start
 * (a serving engine's arena, a memory pool pinned to a budget), or code that runs where even a stream-ordered
 * allocation is unwelcome because its timing must not depend on the state of a pool. It makes no cudaMalloc,
 * cudaMallocAsync, cudaFree or library call that allocates.
 *   - m, n, k as for path 2 (k % 256 == 0, n % 32 == 0, scale arrays 8-byte aligned), and
 *     round_up(m * k, 256) + n * k <= QI_NOALLOC_SCRATCH_BYTES, else QI_NOALLOC_TOO_LARGE and nothing is launched
 *     (64 MiB takes the block's qkv, out and fc1 linears at 4096 rows; fc2, 88 MB, is too large).
 *   - The first call on a device looks up the address of that device's array (cudaGetSymbolAddress, with the device
 *     current) and keeps it; make that call before any stream capture begins.
 *   - One array per device: calls on the same device that overlap in time (different streams or host threads) race
 *     on it. Calls on one stream follow each other and are safe. Nothing in the array has to be cleared.
 * Same bits as qi_w4a4_gemm_ex. No counterpart in the reference (its kernel needs no scratch, gemm.cu:65-189). */
#define QI_NOALLOC_SCRATCH_BYTES (64u << 20)
#define QI_NOALLOC_TOO_LARGE 30001
int qi_w4a4_gemm_noalloc_ex(const void *a_codes, const void *a_scales, const void *w_codes, const void *w_scales,
                            const float *bias, void *y, int y_dtype, long long ldy, int m, int n, int k, void *stream);

/* As qi_w4a4_gemm_ex with the kernel chosen by the caller instead of by shape (for tests and tuning; every path gives
 * the same bits): 0 = by shape; 1 = the int8 kernel that widens the nibbles in shared memory (any k % 128 == 0);
 * 2 = both operands widened to one byte per code in scratch memory, then the byte-operand kernel on CTA pairs
 * (k % 256 == 0, scale arrays 8-byte aligned). Path 2, and path 0 where it chooses path 2 (m, n >= 256 and the
 * conditions of path 2), take (m + n) * k bytes from a memory pool of the library's own (one per device, made at
 * first use, cudaMallocFromPoolAsync) and give them back with cudaFreeAsync, both in stream order; the pool keeps
 * the memory for the next call until qi_w4a4_scratch_trim() returns what is unused to the system. When the pool
 * refuses, path 0 runs path 1 instead. A caller that
 * holds the weights for many calls widens them once (qi_w4a4_widen_codes_ex) and calls qi_w4a4_gemm_wide_ex.
 * No counterpart in the reference (gemm.cu:65-189 is one kernel). */
int qi_w4a4_gemm_path_ex(const void *a_codes, const void *a_scales, const void *w_codes, const void *w_scales,
                         const float *bias, void *y, int y_dtype, long long ldy, int m, int n, int k, int path,
                         void *stream);
int qi_w4a4_scratch_trim(void);

/* qi_f32_to_f16 on a stream. */
int qi_f32_to_f16_ex(const float *source, void *out, unsigned long long count, void *stream);

/* Any m >= 1: rows beyond the last multiple of 128 are handled in the kernel; m <= 8 takes
 * the GEMV path below. */
int qi_w4a16_gemm_ex(const void *x_half, const void *codes, const void *scales, const void *minimums,
                     const float *bias, void *y, int y_dtype, long long ldy, int m, int n, int k, void *stream);

/* 1 <= m <= 8 activation rows (the per-block adaLN modulation linears are m = 1); n % 16 == 0,
 * k % 64 == 0. Same operator as qi_w4a16_gemm without padding m to 128. The reference has no
 * packed m = 1 path (its modulation linear is a BF16 cuBLAS call, transformer.cplus:716-730). */
int qi_w4a16_gemv_ex(const void *x_half, const void *codes, const void *scales, const void *minimums,
                     const float *bias, void *y, int y_dtype, long long ldy, int m, int n, int k, void *stream);

/* `count` matrices of one shape [n, k] against the SAME activations x [m, k], 1 <= m <= 8, in one launch per 64
 * matrices: item i writes y_i [m, ldy] = x . W_i^T (+ bias_i). For the adaLN modulation linears of a denoising step:
 * every block has its own weights and all of them read the same conditioning vector, so the 2 x 60 launches of a
 * step become two (the launch, the first copies and the staging of x are paid once; the weights stream through as
 * one list of tiles). `items` is host memory, read during the call. n % 16 == 0, k % 64 == 0, k <= 4096; codes,
 * scales and minimums of every item 16-byte aligned. Same bits as qi_w4a16_gemv_ex. No counterpart in the reference
 * (its modulation linear is one BF16 cuBLAS call per block, transformer.cplus:716-730). */
typedef struct qi_gemv_item {
    const void *codes, *scales, *minimums; /* [n, k/2] uint8, [n, k/64] float16 each */
    const float *bias;                     /* [n] or NULL */
    void *y;                               /* [m, ldy] of y_dtype */
} qi_gemv_item;
int qi_w4a16_gemv_grouped_ex(const void *x_half, const qi_gemv_item *items, int count, int y_dtype, long long ldy,
                             int m, int n, int k, void *stream);

/* As qi_w4a16_gemm_ex with the tile chosen by the caller instead of by shape (for tests and
 * tuning; every tile gives results within the operator's tolerance, not the same bits):
 * 0 = by shape, 1 = 128x128, 2 = 256x128, 3 = 128x256, 4 = 256x256, 5 = 256x256 on a CTA pair.
 * No counterpart in the reference (gemm.cu:198 has one tile, 128x128x64). */
int qi_w4a16_gemm_tile_ex(const void *x_half, const void *codes, const void *scales, const void *minimums,
                          const float *bias, void *y, int y_dtype, long long ldy, int m, int n, int k, int tile,
                          void *stream);

/* W^[n,k] = fp16(code*scale+minimum) written out as float16 [n,k] (gemm.cu:223-230): the
 * unpacked operand exactly as the GEMM kernels feed it to the tensor cores. */
int qi_w4a16_dequantize_ex(const void *codes, const void *scales, const void *minimums, void *w_half,
                           int n, int k, void *stream);

/* The exact int32 dot of every (row, column, 64-group), dots [m, n, k/64], from the same
 * kernel and tensor-core path as qi_w4a4_gemm (which also still writes y). For checking. */
int qi_w4a4_group_dots_ex(const void *a_codes, const void *a_scales, const void *w_codes, const void *w_scales,
                          float *y, int32_t *dots, int m, int n, int k, void *stream);

/* ---- W4A4 with one byte per code (the fast path on B200) ------------------------------------ */
/* tcgen05 has no 4-bit integer MMA. Codes -7..7 stored one per byte as FP8 E4M3 numbers (exact)
 * go to the tensor cores as they are, and their fp32-accumulated group dots are exact integers
 * (|dot| <= 3136). Weights are widened once when the pack is loaded (qi_w4a4_widen_codes_ex: same
 * integers, twice the bytes of the packed codes); activations come out of the quantiser in this
 * form directly. Scales are the pack's own. Results are the same bits as qi_w4a4_gemm's.
 * None of these has a counterpart in the reference, whose int4 tensor-core path (gemm.cu:60-63)
 * does not exist on this architecture. */

/* codes [rows, k/2] packed nibbles -> bytes [rows, k]; k % 32 == 0. */
int qi_w4a4_widen_codes_ex(const void *codes, void *bytes, long long rows, int k, void *stream);

/* As qi_w4a4_quantize_activations_ex, also writing bytes [m, k]; codes may be NULL. */
int qi_w4a4_quantize_activations_wide_ex(const void *x, int x_dtype, void *codes, void *scales, void *bytes, int m,
                                         int k, void *stream);

/* The activation function that feeds a scheme-6 linear, fused into its quantiser: the same codes, scales and
 * bytes as running the reference's element-wise kernel into an [m, k] float32 matrix and quantising that
 * (the producer's expression is evaluated as the reference writes it), without that matrix in HBM.
 *   qi_w4a4_swiglu_quantize_ex: silu(gate) * up, i.e. qi_swiglu (qwen_image_cuda/cuda/ops.cu:133-145), the
 *     input of the down projection (transformer.cplus:811-813), then qi_w4a4_quantize_activations (gemm.cu:22-57);
 *   qi_w4a4_gelu_quantize_ex: qi_gelu_tanh (ops.cu:155-166), the fc2 input of an MMDiT block, then the same.
 * gate, up, x: [m, k] float32. codes [m, k/2] and bytes [m, k] may each be NULL, not both; scales [m, k/64]. */
int qi_w4a4_swiglu_quantize_ex(const float *gate, const float *up, void *codes, void *scales, void *bytes, int m, int k,
                               void *stream);
int qi_w4a4_gelu_quantize_ex(const float *x, void *codes, void *scales, void *bytes, int m, int k, void *stream);

/* As qi_w4a4_gemm_ex on byte operands a_bytes [m, k], w_bytes [n, k]; k % 128 == 0. */
int qi_w4a4_gemm_wide_ex(const void *a_bytes, const void *a_scales, const void *w_bytes, const void *w_scales,
                         const float *bias, void *y, int y_dtype, long long ldy, int m, int n, int k, void *stream);

/* The same operator on one CTA per 128x128 tile instead of a CTA pair per 256x128 tile (the kernel
 * qi_w4a4_gemm_wide_ex itself falls back to when k is not a multiple of 256 or a scale array is
 * not 8-byte aligned). `dots` may be NULL; otherwise [m, n, k/64] as below. Same bits. */
int qi_w4a4_gemm_wide_single_ex(const void *a_bytes, const void *a_scales, const void *w_bytes, const void *w_scales,
                                const float *bias, void *y, int y_dtype, long long ldy, int32_t *dots, int m, int n,
                                int k, void *stream);

/* As qi_w4a4_group_dots_ex, from the byte-operand kernel. */
int qi_w4a4_group_dots_wide_ex(const void *a_bytes, const void *a_scales, const void *w_bytes, const void *w_scales,
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
    const void *weights_wide; /* scheme 6 only, optional: qi_w4a4_widen_codes_ex(weights) [n, k] bytes */
} qi_packed_linear;

/* The activation arena of transformer.cplus:649-651: codes rows*k_max/2 bytes, code_scales
 * rows*k_max/64*2 bytes, halves rows*k_max*2 bytes. Shared by consecutive linears. */
typedef struct qi_linear_work {
    void *codes;
    void *code_scales;
    void *halves;
    void *wide;           /* optional: rows*k_max bytes; with weights_wide selects the byte-operand W4A4 path */
} qi_linear_work;

/* output[rows, n] = input[rows, k] . W^T for one record. `input` is float32 (the engine's
 * residual stream) unless input_dtype says float16. reuse_input != 0 skips quantising /
 * converting `input` because the previous linear already did so for the same input
 * (q,k,v and gate,up share one: transformer.cplus:760-762,809-810). Returns 1 for an
 * unknown scheme or group size. */
int qi_linear(const qi_packed_linear *record, const qi_linear_work *work, const void *input, int input_dtype,
              void *output, int output_dtype, long long ld_output, int rows, int reuse_input, void *stream);

/* ---- the QIPACK v6 container (host side) ---------------------------------------------------- */
/* A pack is a 256-byte header, a directory of 256-byte records, key=value metadata lines in the padding
 * after the directory, and a data section of 256-byte-aligned regions whose bytes are uploaded verbatim
 * and addressed by file offset (int4_pack.cplus:36-95, 476-518; transformer.cplus:120-123, 569-572).
 * These functions read, check and write that container; they run on the host and touch no GPU.
 * They return 0 or one of the QI_PACK_* codes. Quantising weights is the offline packer's job
 * (qwen-image-quantize, qwen_image_quantize/src/main.cplus:15-55) and is not repeated here. */

#define QI_PACK_IO 20001               /* cannot open, read, write or rename */
#define QI_PACK_NOT_A_PACK 20002       /* magic, header size or tensor count */
#define QI_PACK_POLICY 20003           /* not one of transformer:w4a16-g{32,64,128}-v6, transformer:w4a4-h256-g{..}-v6 */
#define QI_PACK_METADATA 20004         /* metadata outside the directory padding, checksum mismatch, or key not found */
#define QI_PACK_RECORD 20005           /* a record's sizes do not follow from its dimensions, or an unknown scheme */
#define QI_PACK_LAYOUT 20006           /* a region is misaligned, overlaps an earlier one or leaves the file */
#define QI_PACK_TENSOR_CHECKSUM 20007
#define QI_PACK_INVENTORY 20008        /* wrong number of quantised matrices, or bytes after the last region */
#define QI_PACK_PAYLOAD_CHECKSUM 20009
#define QI_PACK_ARGUMENT 20010

typedef struct qi_pack_header_info {
    char policy[33];          /* e.g. "transformer:w4a4-h256-g64-v6" (int4_pack.cplus:107-112) */
    uint32_t scheme;          /* the quantised scheme the policy announces, 0 if none */
    uint32_t tensor_count;
    uint64_t data_offset;     /* file offset of the data section: device address = base + (offset - data_offset) */
    uint64_t file_bytes;
    uint64_t payload_checksum;
} qi_pack_header_info;

typedef struct qi_pack_record_info {  /* int4_pack.cplus:76-95 */
    char name[129];
    uint32_t scheme, rank;
    uint64_t dimensions[4];   /* [0] = outputs n, [1] = inputs k for a matrix */
    uint32_t group_size;
    uint64_t weights_offset, weights_length, scales_offset, scales_length, zeros_offset, zeros_length;
    uint64_t tensor_checksum; /* FNV-1a over weights, scales, zeros in that order */
} qi_pack_record_info;

/* Opens a pack and reads its header, directory and metadata (replaces the reading half of
 * int4_pack.cplus:220-235 and pack_info.cplus:62-145). */
int qi_pack_open(const char *path, void **pack);
int qi_pack_close(void *pack);
int qi_pack_info(void *pack, qi_pack_header_info *info);
int qi_pack_record(void *pack, int index, qi_pack_record_info *info);
/* The value of a metadata line `key=value` (steps, kind, schedule, cache, quant ...: pack_info.cplus:1-5). */
int qi_pack_metadata(void *pack, const char *key, char *value, size_t capacity);
/* `bytes` bytes of the file from `offset` into host memory `out` (for the caller's upload of the data section). */
int qi_pack_read(void *pack, uint64_t offset, uint64_t bytes, void *out);
/* Record `index` as the run-time view the kernels take, for a data section resident at device address
 * `device_data` (what transformer.cplus:569-572 computes per call); QI_PACK_RECORD unless it is a scheme 5 or 6 matrix. */
int qi_pack_linear(void *pack, int index, const void *device_data, struct qi_packed_linear *linear);

/* Everything the reference's verify re-checks (int4_pack.cplus:733-850): policy, metadata placement and checksum,
 * every record's sizes, alignment and order of the regions, every tensor checksum, the inventory and the payload
 * checksum. qi_pack_verify expects the engine's 297 tensors of which 224 quantised matrices, as the reference
 * does; qi_pack_verify_ex takes the expected counts (negative = any). */
int qi_pack_verify(const char *path);
int qi_pack_verify_ex(const char *path, int expected_tensors, int expected_matrices);

/* One tensor in its stored form, for qi_pack_write. A matrix of the pack's quantised scheme carries codes
 * [n, k/2], scales [n, k/group] fp16 and, for scheme 5, zeros (minimums) likewise; anything else is scheme 0
 * (bf16) or 1 (fp16) raw bytes in `weights`. */
typedef struct qi_pack_tensor {
    const char *name;
    uint32_t scheme, rank;
    uint64_t dimensions[4];
    uint32_t group_size;
    const void *weights; uint64_t weights_length;
    const void *scales; uint64_t scales_length;
    const void *zeros; uint64_t zeros_length;
} qi_pack_tensor;

/* Writes a pack: regions laid out as plan_record does (int4_pack.cplus:476-518), checksums as write_from
 * computes them (:628-666), to <path>.tmp, verified, then renamed over `path` (:667-677). `metadata`: the
 * key=value lines, each ending in a newline, or NULL. */
int qi_pack_write(const char *path, const char *policy, const char *metadata, const qi_pack_tensor *tensors, int count);

/* ---- column (N) sharding over the GPUs of one box ------------------------------------------- */
/* No counterpart in the reference, which drives one GPU (qwen_image_cuda/cuda/runtime.cu:6-19).
 * One process per GPU. Rank r of R holds weight rows [r*N/R, (r+1)*N/R) of every region (codes,
 * scales, minimums are per output row, so a shard is a contiguous slice of each), computes
 * y[:, r*N/R:(r+1)*N/R] with the kernels above and the slices are all-gathered with NCCL over
 * NVLink. NCCL is looked up at run time (dlopen of libnccl.so.2, or the path in QI_NCCL_LIBRARY),
 * never linked. Errors of NCCL come back as 10000 + ncclResult_t, a missing NCCL as 10100. */

#define QI_SHARD_ID_BYTES 128

/* Host-only: the rows rank owns. Every shard must be a legal GEMM, so n % (ranks*128) == 0. */
int qi_shard_plan(int n, int ranks, int rank, int *first_row, int *row_count);

/* Rank 0 makes the 128-byte id; the caller carries it to the other ranks by any host channel. */
int qi_shard_unique_id(void *id);

/* Collective over all ranks; the current device becomes the rank's device. */
int qi_shard_create(void **context, int rank, int ranks, const void *id);
int qi_shard_destroy(void *context);
int qi_shard_rank(void *context, int *rank, int *ranks);

/* y_slabs [ranks][rows][n_local] <- every rank's y_local [rows][n_local], on `stream`. */
int qi_shard_all_gather(void *context, const void *y_local, void *y_slabs, int output_dtype, int rows, int n_local,
                        void *stream);

/* qi_linear on this rank's shard (local_record->n = N/R rows) into y_local [rows, N/R], then the
 * all-gather into y_slabs (skipped when y_slabs is NULL or there is one rank). */
int qi_shard_linear(void *context, const qi_packed_linear *local_record, const qi_linear_work *work,
                    const void *input, int input_dtype, void *y_local, void *y_slabs, int output_dtype, int rows,
                    int reuse_input, void *stream);

/* The other split (row-parallel): rank r holds input columns [r*K/R, (r+1)*K/R) of every weight row - a column block
 * of codes [n, K/R/2], scales and minimums [n, K/R/64], copied out of the pack by the caller - and the matching
 * columns of the activations, computes the partial product over its inputs in float32 and the partial results are
 * summed over the ranks (ncclAllReduce, in place): every rank ends with the whole y [rows, n]. It pairs with a
 * column-sharded linear in front of it (fc1 -> activation -> fc2: the column slice a rank computed is the input
 * slice it needs), so that the wide tensor between them is never gathered. K/R must hold whole groups, and for
 * scheme 6 whole 256-input Hadamard blocks; then the slice's activation codes are the unsharded codes' slice. The
 * sum over ranks is a float32 sum in NCCL's order: the result agrees with the unsharded operator to float32
 * rounding of R partial sums, not bit for bit. A bias may be given on rank 0 only. */
int qi_shard_plan_inputs(int k, int scheme, int ranks, int rank, int *first_input, int *input_count);
/* The sum over ranks by itself, in place, on `stream`: y [count] float32 <- sum of every rank's y. For callers that
 * run the partial product themselves (qi_w4a4_gemm_wide_ex and the like on an input slice, float32 output) and want
 * the sum on another stream, under the next linear's kernels. No counterpart in the reference (single GPU). */
int qi_shard_all_reduce_f32(void *context, float *y, unsigned long long count, void *stream);
/* Half of that sum: y [ranks * count_per_rank] float32 on every rank -> y_share [count_per_rank] on rank r = the sum
 * over ranks of y[r * count_per_rank ...] (ncclReduceScatter). For a caller whose next step works on rows - a
 * layer norm, the activation quantiser - and so wants rank r to end with rows [r * rows / R, (r + 1) * rows / R) of a
 * row-parallel linear's output only: half the bytes of the all-reduce cross NVLink. No counterpart in the reference. */
int qi_shard_reduce_scatter_f32(void *context, const float *y, float *y_share, unsigned long long count_per_rank,
                                void *stream);
int qi_shard_linear_inputs(void *context, const struct qi_packed_linear *local_record, const struct qi_linear_work *work,
                           const void *input_local, int input_dtype, float *y, int rows, int reuse_input, void *stream);

/* The W4A4 linear without the all-gather: every rank holds the whole output y [rows, N] and the
 * GEMM stores its slice into every rank's copy itself, over NVLink, from its epilogue.
 *
 * qi_shard_peer_export: `pointer` lies in a cudaMalloc allocation of this process; `handle`
 * (QI_SHARD_PEER_HANDLE_BYTES bytes) and `offset` name it for the other processes of the box, which
 * the caller reaches by any host channel. qi_shard_peer_open, in another process with its own
 * device current, maps that allocation (peer access is enabled on the way) and returns the same
 * address there; qi_shard_peer_close unmaps it. An allocation is opened once per process: carve
 * several outputs out of one allocation on the host. */
#define QI_SHARD_PEER_HANDLE_BYTES 64
int qi_shard_peer_export(const void *pointer, void *handle, size_t *offset);
int qi_shard_peer_open(const void *handle, size_t offset, void **pointer);
int qi_shard_peer_close(void *pointer, size_t offset);

/* y_copies[c][row * ldy + column + j] <- (A . W^T)[row][j] for every copy c < copies (at most 8):
 * qi_w4a4_gemm_wide_ex with the output written to `copies` matrices of the same layout, one of
 * them usually this rank's own and the others peer mappings; `column` (a multiple of 32) is where
 * this rank's slice starts, and a CTA stores to copy first_copy first (give each rank another one).
 * k must be a multiple of 256, n of 32, both scale arrays 8-byte aligned. The stores of a launch
 * are complete when the launch is: a consumer on another rank waits for qi_shard_barrier, placed
 * after the launch in stream order.
 * That barrier orders producers before consumers only. The reverse also needs an order: a copy may
 * be REWRITTEN (by the next step's launch on any rank) only after every rank's readers of it are
 * done. Either queue a second qi_shard_barrier after the readers and before the next writer, or
 * alternate between two sets of copies so that the barrier of step i + 1 (which every rank reaches
 * only after its readers of step i were queued ahead of it in stream order) guards set i. The same
 * rule holds for qi_shard_put_slice. */
int qi_w4a4_gemm_wide_scatter_ex(const void *a_bytes, const void *a_scales, const void *w_bytes, const void *w_scales,
                                 const float *bias, void *const *y_copies, int copies, int first_copy, int y_dtype,
                                 long long ldy, int column, int m, int n, int k, void *stream);

/* The same without a kernel of its own: this rank's slice, columns [column, column + n_local) of its
 * own copy y_copies[rank] (written there by an ordinary GEMM with ldy = N), goes to the same place in
 * every other copy with one 2-D device-to-device copy per GPU, on the copy engines, so that the SMs
 * stay with the next GEMM. Ordered on `stream` like a single operation: it starts after the work
 * queued there before it, and work queued after it starts when all the copies are done. */
int qi_shard_put_slice(void *context, void *const *y_copies, int copies, int output_dtype, long long ldy, int column,
                       int rows, int n_local, void *stream);

/* Every rank's work queued on its `stream` before this call has completed when the call's own work
 * completes on any rank's stream (a four-byte NCCL all-reduce). */
int qi_shard_barrier(void *context, void *stream);

/* ---- diagnostics --------------------------------------------------------------------------- */

/* Kernels of this library never spin without a bound: a wait that runs out records a code
 * (which wait, which stage) and the kernel returns. This reads and clears the code of the
 * current device (0 = healthy). Synchronises the device. */
int qi_kernel_status(unsigned int *status);

/* What the tensor cores of the current device sustain with nothing in their way: every SM issues dense
 * tcgen05.mma instructions (128 x 256 x K) on operands resident in shared memory for about `seconds`
 * (at most 2) and the rate, 2 * multiply-adds per second in units of 1e12, is returned. kind 0: fp16
 * inputs, fp32 accumulators; 1: FP8 E4M3, fp32; 2: int8, int32. Launches on the legacy default stream
 * and synchronises. A measuring aid for rooflines: the reference has nothing like it (its
 * qwen_image_cuda/cuda/bench/bench_gemm_cublas.cu:1-7 times cuBLAS for the same purpose). */
int qi_probe_tensor_rate(int kind, double seconds, double *tera_ops_per_second);

/* Launches one thread that waits, like every wait in this library's kernels, on a barrier that nobody will ever
 * arrive on, with a time limit of `limit_ns` (at most 1e8) instead of the kernels' two seconds. When the limit
 * has passed the thread records 0x0001A000 in the status word and the kernel ends; nothing faults or hangs. For
 * testing what a caller sees after a wait gave up (qi_kernel_status). No counterpart in the reference, whose
 * kernels have no device-side waits (its error convention: gemm.cu:185-188, transformer.cplus:104-110). */
int qi_probe_wait_timeout(unsigned long long limit_ns, void *stream);

/* "qipack_b200 <version> sm_100a" */
const char *qi_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif
