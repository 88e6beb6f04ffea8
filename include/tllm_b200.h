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
#define TLLM_MAX_FUSED        4
#define TLLM_MAX_PEERS        8    /* ranks of a fused all-reduce (one 8-GPU NVSwitch box) */
#define TLLM_AR_MAX_CTAS      256  /* length of the per-rank launch-counter array */    /* matrices per tllm_b200_gemv_packed_multi call */

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


/* ------------------------------------------------------------------------
 * Prepared weights (load-time repack).
 *
 * The streaming tensor-core GEMV reads a kernel-friendly layout: tiles of 16 rows x 128
 * columns, 2 bits per weight (offset codes t + 1 arranged so that one AND makes an MMA
 * operand register), FP16 scales beside them (ternary_llm_b200/csrc/packed_layout.cuh).  It is derived once per
 * matrix at load time from the three reference arrays -- the hook sits right
 * after the reference loader's read_ternary_weight (src/model.cpp:46-60) -- and is
 * lossless for canonical masks (no sign bit without its nonzero bit), which is
 * what the reference's packer writes (ternarize/pack.py:135-138):
 * tllm_b200_weight_unpack returns the original words bit for bit.  A matrix with
 * stray sign bits is refused (TLLM_ERR_NONCANON) and stays on the general path.
 * ------------------------------------------------------------------------ */

/* Size in bytes of the packed form of a [rows, cols] matrix (cols % 128 == 0); rows are
 * padded to a multiple of 16 in it. */
size_t tllm_b200_packed_bytes(int rows, int cols);

/*
 * Repack into `packed` (device, 16-byte aligned, >= tllm_b200_packed_bytes).
 * Runs on `stream` and SYNCHRONISES it before returning (a load-time call).
 * The first call on a device allocates the library's per-device scratch.
 */
int tllm_b200_weight_prepare(const uint32_t* nonzero_masks, const uint32_t* sign_masks,
                             const void* scales, int rows, int cols, int group_size,
                             void* packed, size_t packed_size, void* stream);

/* Inverse of prepare: writes canonical nonzero/sign words and the scales. */
int tllm_b200_weight_unpack(const void* packed, int rows, int cols, int group_size,
                            uint32_t* nonzero_masks, uint32_t* sign_masks, void* scales,
                            void* stream);

/*
 * Associates a prepared buffer with the reference arrays it was made from, keyed
 * by the nonzero_masks pointer: afterwards tllm_b200_gemv, _gemv_batched,
 * _gemv_int8 and _gemm called with that pointer and the same rows/cols use the
 * prepared weights, so the reference's call sites
 * (src/transformer.cpp:102-143,199-217,264-278) need no change.  Unregister
 * before freeing either buffer (reference Model::free_gpu, src/model.cpp:221-250).
 */
int tllm_b200_weight_register(const uint32_t* nonzero_masks, const void* packed, int rows, int cols);
int tllm_b200_weight_unregister(const uint32_t* nonzero_masks);

/*
 * GEMV directly on prepared weights; same arithmetic contract as tllm_b200_gemv /
 * _gemv_batched / _gemv_int8.  These kernels keep partial sums of row blocks that
 * span two SMs in a per-device scratch that the library allocates at its first
 * use on a device (make one call per device before capturing a CUDA graph).
 * FP16 activations are converted per scale group to block fixed point and the
 * group sums are exact integers: 24 bits below the group's largest magnitude for
 * one or two vectors per call, 16 bits for passes of three or four vectors (their
 * rounding error per output is at most 2^-17 * sum over groups of scale * 128 *
 * max|x| of the group, under half of the 2e-3 * sum|scale * x| bound for any
 * input); nine vectors and more run on the tcgen05 GEMM kernel in FP16.
 */
int tllm_b200_gemv_packed(const void* packed, const void* x, void* y,
                          int batch, int rows, int cols, void* stream);
int tllm_b200_gemv_int8_packed(const void* packed, const int8_t* input_int8, float input_scale,
                               void* y, int rows, int cols, void* stream);

/*
 * y_i = W_i x for `count` (1..TLLM_MAX_FUSED) prepared matrices that share the FP16
 * activation vector x and the column count -- q/k/v after the attention norm, gate/up
 * after the FFN norm (the reference issues them as separate calls on the same input,
 * src/transformer.cpp:206-222,271-283).  One launch streams all of them, so small
 * matrices (k, v) no longer pay a launch each; results equal those of `count` calls
 * of tllm_b200_gemv_packed up to the order of the FP32 additions over K.  packed, y, rows
 * are HOST arrays of length count.
 * Fastest when the matrices were packed back to back -- packed[i+1] == packed[i] +
 * tllm_b200_packed_bytes(rows[i], cols) with every rows[i] but the last a multiple of 16
 * (prepare them into consecutive pieces of one buffer): they are then streamed as ONE
 * matrix in one launch.  Otherwise one launch per matrix.
 */
int tllm_b200_gemv_packed_multi(int count, const void* const* packed, void* const* y, const int* rows,
                                int cols, const void* x, void* stream);

/* The same with the shared input vector made inside the kernel: x = rmsnorm(a (+ b)) *
 * norm_weight with the arithmetic of add_forward followed by rmsnorm_forward
 * (include/kernels.cuh:45-48,64-66: FP16-rounded sum, FP32 mean of squares of the rounded
 * values, one FP16 rounding), what the reference does with a residual add and an rmsnorm
 * launch in front of its q/k/v and gate/up projections (src/transformer.cpp:199-217,264-278).  b may be NULL (no residual).  res_out (may be NULL)
 * receives the rounded sum a + b and must not alias a or b.  The matrices must be packed back
 * to back (count > 1).  a, b, norm_weight, res_out: FP16 [cols], 16-byte aligned. */
int tllm_b200_gemv_packed_multi_norm(int count, const void* const* packed, void* const* y, const int* rows, int cols,
                                     const void* a, const void* b, const void* norm_weight, void* res_out, float eps,
                                     void* stream);

/*
 * Row-parallel GEMV of a tensor-parallel layer (o_proj, down_proj: each rank holds a
 * 128-aligned K range of the matrix and the matching slice of x) with the all-reduce
 * FUSED into the kernel: every rank runs this call on its shard; each CTA stores its
 * FP32 partial sums into all ranks' receive buffers over NVLink as 8-byte {value, launch
 * number} words (plain peer stores; the launch number is the arrival flag, so there is no
 * fence and no separate flag round), polls -- bounded -- its OWN memory for the other
 * ranks' words of the same rows, adds the contributions in rank order and writes the FP16
 * result y[rows], identical on all ranks.  No counterpart in the reference (which is
 * single-GPU); it replaces GEMV + ncclAllReduce.
 *   peer_recv[d] : rank d's receive buffer, 8-byte words [2][world][rows_max], as mapped in
 *                  THIS process (peer / symmetric memory), zeroed before first use
 *   epoch_local  : this rank's launch counters, uint32 [TLLM_AR_MAX_CTAS], zeroed
 * All ranks must issue the same sequence of these calls.  Each CTA owns whole 16-row
 * blocks.  A wait that expires sets
 * the device error flag (tllm_b200_check_device_errors); after the first one that expires
 * in a CTA, its remaining waits of that launch return at once.
 */
int tllm_b200_gemv_packed_allreduce(const void* packed, const void* x, void* y, int rows, int cols,
                                    int rank, int world, void* const* peer_recv, void* epoch_local,
                                    int rows_max, void* stream);

/*
 * Time stamps of the fused all-reduce, for finding out where a tensor-parallel step spends
 * its time.  While a buffer is set for the current device, CTA 0 of every
 * tllm_b200_gemv_packed_allreduce launch on it writes a record of eight 64-bit words to
 * buffer[(e % records) * 8 ..], e being the launch number: the GPU's nanosecond timer at
 * {kernel entry, end of the stream-order wait, partial sums ready, peer stores issued, all
 * ranks' words seen and summed}, then e, then two unused words.  buffer: device memory of
 * records * 64 bytes, owned by the caller; NULL switches the stamps off (the default).  Costs
 * a few instructions per launch.  No counterpart in the reference.
 */
int tllm_b200_allreduce_trace(void* buffer, int records);

/*
 * tllm_b200_gemv_packed for one FP16 vector, for callers that cannot let a library
 * allocate device memory (a server that owns all of HBM through its own arena, a
 * real-time loop, a host that audits allocations up front).  It has no counterpart
 * in the reference.  Nothing is allocated, by this call or any routine it uses: the
 * split-K scratch is a fixed 40 KB array inside the library image, present on every
 * GPU that loads the library until the process exits.
 * Limits: rows <= 65536 (TLLM_ERR_SIZE beyond), cols as for tllm_b200_gemv_packed.
 * The first call on a device resolves the array's device address and configures the
 * kernel; make that first call before any stream capture.  All calls share the one
 * array and it keeps the last call's contents (its records are cleared on
 * `stream` before each launch): calls whose kernels overlap on the GPU, for example
 * from two streams, race with each other -- serialise them.
 */
int tllm_b200_gemv_packed_noalloc(const void* packed, const void* x, void* y,
                                  int rows, int cols, void* stream);

/*
 * Error report for tllm_b200_gemv_packed_noalloc, equally allocation-free (the regular
 * tllm_b200_check_device_errors reads a flag in the library's allocated scratch and may
 * set that scratch up).  SYNCHRONISES `stream`, returns TLLM_ERR_TIMEOUT if a bounded wait
 * of a no-allocation launch expired since the last check (and clears the flag, which lives
 * in the same fixed array), else TLLM_OK.  No counterpart in the reference.
 */
int tllm_b200_gemv_packed_noalloc_status(void* stream);

/*
 * Prefill GEMM on prepared weights: C[M,N] = A[M,K] . W^T, same contract as
 * tllm_b200_gemm.  M > 8 runs the tcgen05 tensor-core kernel (weights expanded to
 * exact FP16 {-s,0,+s} in tensor memory, FP32 accumulation in TMEM; token tile 32, 64,
 * 128 or 256 by M); smaller M runs passes of the streaming GEMV.  tllm_b200_gemm reaches the same kernels when
 * the weight pointer has been registered.
 */
int tllm_b200_gemm_packed(const void* A, const void* packed, void* C, int M, int N, int K, void* stream);

/*
 * Device-side waits in the kernels are bounded; one that expires sets a flag on
 * the device and the kernel returns early (its output is then invalid).  This
 * call SYNCHRONISES `stream`, returns TLLM_ERR_TIMEOUT if the flag was set since
 * the last check (and clears it), else TLLM_OK.  No counterpart in the reference,
 * which checks no errors.
 */
int tllm_b200_check_device_errors(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TLLM_B200_H */
