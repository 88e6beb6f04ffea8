/*
 * tllm_b200 -- B200 (sm_100a) implementation of the ternary weight-contraction
 * path of jastaq/ternary-llm, behind a plain C ABI.
 *
 * Every pointer is a DEVICE pointer unless the comment says otherwise, owned by
 * the caller; `stream` is a cudaStream_t passed as void* (NULL = legacy default
 * stream, which is what the reference's call sites use).  Every function returns
 * TLLM_OK (0) or a negative status and never allocates, except where stated.
 * The reference interface returns void and checks nothing; the C++ shim that
 * re-exports the reference's names (ternary::ternary_gemv ...) prints the status
 * text to stderr when a call fails.
 *
 * Weight encoding (reference ternarize/pack.py:120-169, include/model.h:12-22):
 *   nonzero_masks, sign_masks : uint32 [rows, cols/32] row-major; bit k of word c
 *       of row r is weight [r, 32c+k]; value = nz ? (sign ? +1 : -1) : 0.
 *       A sign bit whose nonzero bit is clear decodes to 0.
 *   scales : IEEE binary16 [rows, cols/group_size] row-major, any sign.
 * Constraints: group_size == 128, cols % 128 == 0, rows >= 1; mask and scale
 * pointers 16-byte aligned (cudaMalloc gives 256), activations/outputs 2-byte.
 */
#ifndef TLLM_B200_H
#define TLLM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TLLM_OK               0
#define TLLM_ERR_NULL        -1   /* a required pointer is NULL                  */
#define TLLM_ERR_ALIGN       -2   /* a pointer is not aligned as required        */
#define TLLM_ERR_SHAPE       -3   /* rows/cols/M/N/K out of range, cols % 128    */
#define TLLM_ERR_GROUP       -4   /* group_size != 128                           */
#define TLLM_ERR_BATCH       -5   /* batch outside 1..TLLM_MAX_BATCH             */
#define TLLM_ERR_LAUNCH      -6   /* CUDA reported a launch/runtime error        */
#define TLLM_ERR_DEVICE      -7   /* current device is not compute capability 10 */
#define TLLM_ERR_NONCANON    -8   /* prepare: a sign bit is set without its nonzero bit */
#define TLLM_ERR_SIZE        -9   /* a caller buffer is too small / size over a stated maximum */
#define TLLM_ERR_TIMEOUT     -10  /* a bounded device-side wait gave up          */

#define TLLM_GROUP_SIZE       128
#define TLLM_MAX_BATCH        16

/* Text for a status code; never NULL. */
const char* tllm_b200_status_string(int status);
/* Detail of the last failure on the calling thread ("" if none). */
const char* tllm_b200_last_error(void);
/* 1000*major + minor of this library. */
int tllm_b200_version(void);

/*
 * Decode GEMV, FP16 activations:  y[n] = sum_g scale[n,g] * sum_{k in g} t[n,k] * x[k],
 * FP32 accumulation, FP16 result.
 * Replaces ternary::ternary_gemv, reference include/kernels.cuh:11-14
 * (kernels/ternary_gemv.cu:27-100).  x: half[cols], y: half[rows].
 */
int tllm_b200_gemv(const uint32_t* nonzero_masks, const uint32_t* sign_masks,
                   const void* scales, const void* x, void* y,
                   int rows, int cols, int group_size, void* stream);

/*
 * The same contraction for `batch` activation vectors in ONE pass over the
 * weights: x half[batch, cols] row-major, y half[batch, rows] row-major,
 * 1 <= batch <= TLLM_MAX_BATCH.  Extension of include/kernels.cuh:11-14; it is
 * what ternary::ternary_gemm (include/kernels.cuh:37-40) forwards to when
 * M <= TLLM_MAX_BATCH.
 */
int tllm_b200_gemv_batched(const uint32_t* nonzero_masks, const uint32_t* sign_masks,
                           const void* scales, const void* x, void* y,
                           int batch, int rows, int cols, int group_size, void* stream);

/*
 * Decode GEMV, INT8 activations: y[n] = input_scale * sum_g scale[n,g] * S[n,g]
 * with S the exact integer group sum of t[n,k]*xq[k].  input_scale is a host
 * float by value, as in the reference.
 * Replaces ternary::ternary_gemv_int8, include/kernels.cuh:19-24
 * (kernels/ternary_gemv.cu:116-216).  xq: int8[cols], y: half[rows].
 */
int tllm_b200_gemv_int8(const uint32_t* nonzero_masks, const uint32_t* sign_masks,
                        const void* weight_scales, const int8_t* input_int8,
                        float input_scale, void* y,
                        int rows, int cols, int group_size, void* stream);

/*
 * Per-vector absmax quantisation half[n] -> int8[n] + one float scale on the
 * device: scale = absmax/127 (1.0 when absmax == 0),
 * q = clamp(rint(x * 127/absmax), -127, 127), ties to even.
 * Replaces ternary::quantize_absmax_int8, include/kernels.cuh:30-32
 * (kernels/activations.cu:88-151).
 */
int tllm_b200_quantize_absmax_int8(const void* x, int8_t* q, float* scale,
                                   int n, void* stream);

/*
 * Prefill GEMM: C[M,N] = A[M,K] . W^T, A and C row-major FP16, W the ternary
 * matrix [N,K] with its per-group scales; FP32 accumulation.
 * Replaces ternary::ternary_gemm, include/kernels.cuh:37-40
 * (kernels/ternary_gemm.cu:33-195).
 */
int tllm_b200_gemm(const void* A, const uint32_t* nz_B, const uint32_t* sign_B,
                   const void* scales_B, void* C,
                   int M, int N, int K, int group_size, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TLLM_B200_H */
