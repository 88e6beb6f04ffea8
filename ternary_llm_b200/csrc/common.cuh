// Shared declarations for the tllm_b200 CUDA sources (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "tllm_b200.h"

namespace tllm {

constexpr int kGroup = TLLM_GROUP_SIZE;   // weights per scale group along K
constexpr int kMaxBatch = TLLM_MAX_BATCH;

// Records a message for tllm_b200_last_error() and returns `status`.
int fail(int status, const char* fmt, ...);
// cudaPeekAtLastError -> status (does not clear sticky errors, does not sync).
int check_launch(const char* what);
// TLLM_OK when the current device is compute capability 10.x, else TLLM_ERR_DEVICE.
int check_device();

// ---- launchers implemented in the kernel translation units ----------------
// General-shape SIMT kernels on the reference layout (any rows >= 1).
int launch_gemv_simt(const uint32_t* nz, const uint32_t* sg, const half* scales,
                     const half* x, half* y, int batch, int rows, int cols,
                     cudaStream_t stream);
int launch_gemv_int8_simt(const uint32_t* nz, const uint32_t* sg, const half* scales,
                          const int8_t* xq, float input_scale, half* y, int rows, int cols,
                          cudaStream_t stream);
int launch_quantize_absmax_int8(const half* x, int8_t* q, float* scale, int n,
                                cudaStream_t stream);

// Tensor-core streaming kernels on the packed layout (gemv_mma.cu).
size_t packed_bytes(int rows, int cols);
// Row counts that are a multiple of this pack without padding (matrices packed back to back
// can then be streamed as one).
int packed_row_align();
const uint8_t* lookup_packed(const void* nz, int rows, int cols);
int launch_gemv_packed(const uint8_t* packed, const half* x, half* y, int batch, int rows, int cols,
                       cudaStream_t stream);
int launch_gemv_int8_packed(const uint8_t* packed, const int8_t* xq, float in_scale, half* y, int rows,
                            int cols, cudaStream_t stream);
int weight_prepare(const uint32_t* nz, const uint32_t* sg, const half* scales, int rows, int cols,
                   uint8_t* packed, cudaStream_t stream);
int weight_unpack(const uint8_t* packed, int rows, int cols, uint32_t* nz, uint32_t* sg, half* scales,
                  cudaStream_t stream);
int weight_register(const void* nz, const uint8_t* packed, int rows, int cols);
int weight_unregister(const void* nz);
int device_error_check(cudaStream_t stream);
// Device error flag of the current device (nullptr if the library scratch cannot be set up).
int* device_error_flag();
int launch_gemv_packed_allreduce(const uint8_t* packed, const half* x, half* y, int rows, int cols, int rank,
                                 int world, void* const* peer_recv, void* epoch_local, int rows_max,
                                 cudaStream_t stream);
int allreduce_set_trace(void* buffer, int records);
int launch_gemv_packed_multi(int count, const uint8_t* const* packed, half* const* y, const int* rows, int cols,
                             const half* x, cudaStream_t stream);
int launch_gemv_int8_packed_multi(int count, const uint8_t* const* packed, half* const* y, const int* rows,
                                  int cols, const int8_t* xq, const float* scale_dev, cudaStream_t stream);
// INT8 GEMVs that build their activation vector inside the kernel from FP16 inputs:
//   norm: x = quantise(rmsnorm(a (+ b)) * w), half(a + b) stored to res_out (may be null)
//   silu: x = quantise(silu(gate) * up)
//   quant: x = quantise(x_f16)
int launch_gemv_packed_multi_norm(int count, const uint8_t* const* packed, half* const* y, const int* rows, int cols,
                                  const half* a, const half* b, const half* w, half* res_out, float eps,
                                  cudaStream_t stream);
int launch_gemv_int8_packed_norm(const uint8_t* packed, const half* a, const half* b, const half* w, half* res_out,
                                 float eps, half* y, int rows, int cols, cudaStream_t stream);
int launch_gemv_int8_packed_silu(const uint8_t* packed, const half* gate, const half* up, half* y, int rows, int cols,
                                 cudaStream_t stream);
int launch_gemv_int8_packed_quant(const uint8_t* packed, const half* x, half* y, int rows, int cols, cudaStream_t stream);
int launch_gemv_packed_noalloc(const uint8_t* packed, const half* x, half* y, int rows, int cols,
                               cudaStream_t stream);
int noalloc_error_check(cudaStream_t stream);

// tcgen05 prefill GEMM on prepared weights (gemm_tcgen05.cu).
bool gemm_tcgen05_supported(int M, int N, int K);
int launch_gemm_tcgen05(const half* A, const uint8_t* packed, half* C, int M, int N, int K, cudaStream_t stream);

// ---- small device helpers --------------------------------------------------
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

}  // namespace tllm
