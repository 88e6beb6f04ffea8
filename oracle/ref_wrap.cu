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

}
