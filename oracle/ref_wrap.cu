/*
 * extern "C" handles onto the UNMODIFIED reference sources, compiled where they
 * lie (never copied): TEST INFRASTRUCTURE, built only by oracle/Makefile into
 * oracle/_ref/libref.so.
 *
 *   ref_cpu_reference      -> cpu_reference        tests/test_ternary_gemv.cu:40-75
 *   ref_ternary_gemv       -> ternary::ternary_gemv        kernels/ternary_gemv.cu:89-100
 *   ref_ternary_gemv_int8  -> ternary::ternary_gemv_int8   kernels/ternary_gemv.cu:201-216
 *   ref_quantize_absmax_int8 -> ternary::quantize_absmax_int8  kernels/activations.cu:144-151
 *   ref_ternary_gemm       -> ternary::ternary_gemm        kernels/ternary_gemm.cu:178-195
 *   ref_rmsnorm_forward, ref_rope_forward, ref_attention_forward, ref_silu_mul_forward,
 *   ref_add_forward, ref_embedding_lookup, ref_copy_to_kv_cache, ref_fp16_gemv, ref_fp16_gemm
 *                          -> the functions of the same names in kernels/rmsnorm.cu, rope.cu,
 *                             attention.cu, activations.cu, elementwise.cu
 *
 * The GPU entry points take device pointers and a stream and launch the
 * reference's own kernels (compiled here for sm_100); they serve as a second
 * checker and as a timed baseline on the GPU, never as part of the library.
 */
#include "kernels.cuh"

void cpu_reference(const uint32_t*, const uint32_t*, const float*, const float*,
                   float*, int, int, int);

extern "C" {

void ref_cpu_reference(const uint32_t* nz, const uint32_t* sg, const float* scales,
                       const float* x, float* y, int rows, int cols, int gs)
{
    cpu_reference(nz, sg, scales, x, y, rows, cols, gs);
}

int ref_ternary_gemv(const void* nz, const void* sg, const void* scales, const void* x,
                     void* y, int rows, int cols, int gs, void* stream)
{
    ternary::ternary_gemv((const uint32_t*)nz, (const uint32_t*)sg, (const half*)scales,
                          (const half*)x, (half*)y, rows, cols, gs, (cudaStream_t)stream);
    return (int)cudaPeekAtLastError();
}

int ref_ternary_gemv_int8(const void* nz, const void* sg, const void* scales, const void* xq,
                          float input_scale, void* y, int rows, int cols, int gs, void* stream)
{
    ternary::ternary_gemv_int8((const uint32_t*)nz, (const uint32_t*)sg, (const half*)scales,
                               (const int8_t*)xq, input_scale, (half*)y, rows, cols, gs,
                               (cudaStream_t)stream);
    return (int)cudaPeekAtLastError();
}

int ref_quantize_absmax_int8(const void* x, void* q, void* scale, int n, void* stream)
{
    ternary::quantize_absmax_int8((const half*)x, (int8_t*)q, (float*)scale, n,
                                  (cudaStream_t)stream);
    return (int)cudaPeekAtLastError();
}

int ref_ternary_gemm(const void* a, const void* nz, const void* sg, const void* scales, void* c,
                     int m, int n, int k, int gs, void* stream)
{
    ternary::ternary_gemm((const half*)a, (const uint32_t*)nz, (const uint32_t*)sg,
                          (const half*)scales, (half*)c, m, n, k, gs, (cudaStream_t)stream);
    return (int)cudaPeekAtLastError();
}


int ref_rmsnorm_forward(const void* in, const void* w, void* out, const void* res, void* res_out, int batch,
                        int dim, float eps, void* stream)
{
    ternary::rmsnorm_forward((const half*)in, (const half*)w, (half*)out, (const half*)res, (half*)res_out, batch,
                             dim, eps, (cudaStream_t)stream);
    return (int)cudaPeekAtLastError();
}

int ref_rope_forward(void* q, void* k, int batch, int seq_len, int n_heads, int n_kv_heads, int head_dim,
                     int start_pos, float theta, void* stream)
{
    ternary::rope_forward((half*)q, (half*)k, batch, seq_len, n_heads, n_kv_heads, head_dim, start_pos, theta,
                          (cudaStream_t)stream);
    return (int)cudaPeekAtLastError();
}

int ref_attention_forward(const void* q, const void* kc, const void* vc, void* out, int batch, int n_heads,
                          int n_kv_heads, int head_dim, int seq_len, int kv_len, int kv_len_max, void* stream)
{
    ternary::attention_forward((const half*)q, (const half*)kc, (const half*)vc, (half*)out, batch, n_heads,
                               n_kv_heads, head_dim, seq_len, kv_len, kv_len_max, (cudaStream_t)stream);
    return (int)cudaPeekAtLastError();
}

int ref_silu_mul_forward(const void* gate, const void* up, void* out, int size, void* stream)
{
    ternary::silu_mul_forward((const half*)gate, (const half*)up, (half*)out, size, (cudaStream_t)stream);
    return (int)cudaPeekAtLastError();
}

int ref_add_forward(const void* a, const void* b, void* out, int size, void* stream)
{
    ternary::add_forward((const half*)a, (const half*)b, (half*)out, size, (cudaStream_t)stream);
    return (int)cudaPeekAtLastError();
}

int ref_embedding_lookup(const void* table, const int* idx, void* out, int n_tokens, int dim, void* stream)
{
    ternary::embedding_lookup((const half*)table, idx, (half*)out, n_tokens, dim, (cudaStream_t)stream);
    return (int)cudaPeekAtLastError();
}

int ref_copy_to_kv_cache(const void* k, const void* v, void* kc, void* vc, int batch, int n_kv_heads, int head_dim,
                         int seq_len, int start_pos, int max_seq_len, void* stream)
{
    ternary::copy_to_kv_cache((const half*)k, (const half*)v, (half*)kc, (half*)vc, batch, n_kv_heads, head_dim,
                              seq_len, start_pos, max_seq_len, (cudaStream_t)stream);
    return (int)cudaPeekAtLastError();
}

int ref_fp16_gemv(const void* w, const void* x, void* y, int rows, int cols, void* stream)
{
    ternary::fp16_gemv((const half*)w, (const half*)x, (half*)y, rows, cols, (cudaStream_t)stream);
    return (int)cudaPeekAtLastError();
}

int ref_fp16_gemm(const void* a, const void* b, void* c, int m, int n, int k, void* stream)
{
    ternary::fp16_gemm((const half*)a, (const half*)b, (half*)c, m, n, k, (cudaStream_t)stream);
    return (int)cudaPeekAtLastError();
}

}
