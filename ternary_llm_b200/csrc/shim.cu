// C++ names of the reference's operator interface, forwarding to the C ABI.
//
// The reference engine (src/transformer.cpp:107,112,132,139,201-217,266-278) and
// its tests call four free functions in namespace `ternary` declared in its
// include/kernels.cuh:11-40, with C++ linkage, void return and a trailing stream
// defaulted to 0.  Defining the same four signatures here lets that code link
// against this library in place of kernels/ternary_gemv.cu, kernels/ternary_gemm.cu
// and the quantiser in kernels/activations.cu, unmodified.  The reference
// interface cannot report an error, so a failed call prints its status.
#include <cstdio>

#include "common.cuh"

namespace ternary {

static void report(const char* fn, int st)
{
    if (st != TLLM_OK)
        fprintf(stderr, "[tllm_b200] %s failed: %s (%s)\n", fn, tllm_b200_status_string(st),
                tllm_b200_last_error());
}

void ternary_gemv(const uint32_t* nonzero_masks, const uint32_t* sign_masks, const half* scales,
                  const half* input, half* output, int rows, int cols, int group_size,
                  cudaStream_t stream)
{
    report("ternary_gemv", tllm_b200_gemv(nonzero_masks, sign_masks, scales, input, output, rows, cols,
                                          group_size, stream));
}

void ternary_gemv_int8(const uint32_t* nonzero_masks, const uint32_t* sign_masks,
                       const half* weight_scales, const int8_t* input_int8, float input_scale,
                       half* output, int rows, int cols, int group_size, cudaStream_t stream)
{
    report("ternary_gemv_int8",
           tllm_b200_gemv_int8(nonzero_masks, sign_masks, weight_scales, input_int8, input_scale, output,
                               rows, cols, group_size, stream));
}

void quantize_absmax_int8(const half* input, int8_t* output, float* scale, int n, cudaStream_t stream)
{
    report("quantize_absmax_int8", tllm_b200_quantize_absmax_int8(input, output, scale, n, stream));
}

void ternary_gemm(const half* A, const uint32_t* nz_B, const uint32_t* sign_B, const half* scales_B,
                  half* C, int M, int N, int K, int group_size, cudaStream_t stream)
{
    report("ternary_gemm", tllm_b200_gemm(A, nz_B, sign_B, scales_B, C, M, N, K, group_size, stream));
}

}  // namespace ternary
