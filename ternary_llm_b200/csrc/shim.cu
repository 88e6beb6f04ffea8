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

// The other operators of the reference interface (its include/kernels.cuh:45-84), so that
// the engine can link against this library with none of the reference's kernels.  When
// the reference's own definitions are linked into the executable as well, the
// executable's take precedence and these stay unused.
#include "tllm_b200_layer.h"

namespace ternary {

void rmsnorm_forward(const half* input, const half* weight, half* output, const half* residual, half* residual_out,
                     int batch, int dim, float eps, cudaStream_t stream)
{
    report("rmsnorm_forward", tllm_b200_rmsnorm(input, weight, output, residual, residual_out, batch, dim, eps, stream));
}

void rope_forward(half* q, half* k, int batch, int seq_len, int n_heads, int n_kv_heads, int head_dim, int start_pos,
                  float theta, cudaStream_t stream)
{
    report("rope_forward", tllm_b200_rope(q, k, batch, seq_len, n_heads, n_kv_heads, head_dim, start_pos, theta, stream));
}

void attention_forward(const half* q, const half* k_cache, const half* v_cache, half* output, int batch, int n_heads,
                       int n_kv_heads, int head_dim, int seq_len, int kv_len, int kv_len_max, cudaStream_t stream)
{
    report("attention_forward", tllm_b200_attention(q, k_cache, v_cache, output, batch, n_heads, n_kv_heads, head_dim,
                                                    seq_len, kv_len, kv_len_max, stream));
}

void silu_mul_forward(const half* gate, const half* up, half* output, int size, cudaStream_t stream)
{
    report("silu_mul_forward", tllm_b200_silu_mul(gate, up, output, size, stream));
}

void add_forward(const half* a, const half* b, half* output, int size, cudaStream_t stream)
{
    report("add_forward", tllm_b200_add(a, b, output, size, stream));
}

void embedding_lookup(const half* table, const int* indices, half* output, int n_tokens, int dim, cudaStream_t stream)
{
    report("embedding_lookup", tllm_b200_embedding_lookup(table, indices, output, n_tokens, dim, stream));
}

void copy_to_kv_cache(const half* k, const half* v, half* k_cache, half* v_cache, int batch, int n_kv_heads,
                      int head_dim, int seq_len, int start_pos, int max_seq_len, cudaStream_t stream)
{
    report("copy_to_kv_cache", tllm_b200_copy_to_kv_cache(k, v, k_cache, v_cache, batch, n_kv_heads, head_dim, seq_len,
                                                          start_pos, max_seq_len, stream));
}

void fp16_gemv(const half* weight, const half* input, half* output, int rows, int cols, cudaStream_t stream)
{
    report("fp16_gemv", tllm_b200_fp16_gemv(weight, input, output, rows, cols, stream));
}

void fp16_gemm(const half* A, const half* B, half* C, int M, int N, int K, cudaStream_t stream)
{
    report("fp16_gemm", tllm_b200_fp16_gemm(A, B, C, M, N, K, stream));
}

}  // namespace ternary
