// Per-vector absmax INT8 quantisation, half[n] -> int8[n] + float scale.
//
// Semantics of the reference kernels/activations.cu:88-142: absmax in FP32;
// scale = absmax/127, or 1.0 for an all-zero vector; q = clamp(rint(x * (127 /
// absmax)), -127, 127) with round-half-even.  The vector (at most a few tens of
// thousands of elements) is handled by one CTA of 1024 threads: it is read once
// with 128-bit loads into registers/shared memory, reduced, and quantised from
// the staged copy, so global memory is read once instead of twice.
#include "common.cuh"

namespace tllm {

constexpr int kQuantThreads = 1024;
constexpr int kQuantStage = 32768;   // halves kept in shared memory (64 KB)

__global__ void __launch_bounds__(kQuantThreads)
quantize_absmax_int8_kernel(const half* __restrict__ x, int8_t* __restrict__ q,
                            float* __restrict__ out_scale, int n)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    half* stage = reinterpret_cast<half*>(smem_raw);
    __shared__ float warp_part[kQuantThreads / 32];
    __shared__ float s_absmax;

    const int tid = threadIdx.x;
    const int staged = n < kQuantStage ? n : kQuantStage;
    const bool vec = ((reinterpret_cast<uintptr_t>(x) & 15) == 0);

    float m = 0.f;
    if (vec) {
        const int n8 = staged / 8;
        const uint4* x4 = reinterpret_cast<const uint4*>(x);
        for (int i = tid; i < n8; i += kQuantThreads) {
            const uint4 v = __ldg(x4 + i);
            reinterpret_cast<uint4*>(stage)[i] = v;
            const half2* h = reinterpret_cast<const half2*>(&v);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 f = __half22float2(h[j]);
                m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
            }
        }
        for (int i = n8 * 8 + tid; i < staged; i += kQuantThreads) {
            const half v = x[i];
            stage[i] = v;
            m = fmaxf(m, fabsf(__half2float(v)));
        }
    } else {
        for (int i = tid; i < staged; i += kQuantThreads) {
            const half v = x[i];
            stage[i] = v;
            m = fmaxf(m, fabsf(__half2float(v)));
        }
    }
    for (int i = staged + tid; i < n; i += kQuantThreads)      // tail beyond the staged part
        m = fmaxf(m, fabsf(__half2float(x[i])));

    m = warp_max(m);
    if ((tid & 31) == 0) warp_part[tid >> 5] = m;
    __syncthreads();
    if (tid < 32) {
        float v = warp_part[tid];
        v = warp_max(v);
        if (tid == 0) {
            s_absmax = v;
            *out_scale = (v > 0.f) ? (v / 127.0f) : 1.0f;
        }
    }
    __syncthreads();
    const float absmax = s_absmax;
    const float inv = (absmax > 0.f) ? (127.0f / absmax) : 0.f;

    const bool qvec = ((reinterpret_cast<uintptr_t>(q) & 3) == 0);
    if (qvec) {
        const int n4 = staged / 4;
        for (int i = tid; i < n4; i += kQuantThreads) {
            const uint2 v = reinterpret_cast<const uint2*>(stage)[i];
            const float2 a = __half22float2(*reinterpret_cast<const half2*>(&v.x));
            const float2 b = __half22float2(*reinterpret_cast<const half2*>(&v.y));
            const int q0 = max(-127, min(127, __float2int_rn(a.x * inv)));
            const int q1 = max(-127, min(127, __float2int_rn(a.y * inv)));
            const int q2 = max(-127, min(127, __float2int_rn(b.x * inv)));
            const int q3 = max(-127, min(127, __float2int_rn(b.y * inv)));
            reinterpret_cast<uint32_t*>(q)[i] =
                (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) |
                ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
        }
        for (int i = n4 * 4 + tid; i < staged; i += kQuantThreads)
            q[i] = (int8_t)max(-127, min(127, __float2int_rn(__half2float(stage[i]) * inv)));
    } else {
        for (int i = tid; i < staged; i += kQuantThreads)
            q[i] = (int8_t)max(-127, min(127, __float2int_rn(__half2float(stage[i]) * inv)));
    }
    for (int i = staged + tid; i < n; i += kQuantThreads)
        q[i] = (int8_t)max(-127, min(127, __float2int_rn(__half2float(x[i]) * inv)));
}

int launch_quantize_absmax_int8(const half* x, int8_t* q, float* scale, int n, cudaStream_t stream)
{
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const size_t smem = (size_t)kQuantStage * sizeof(half);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaFuncSetAttribute(quantize_absmax_int8_kernel,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        // same carve-out as the GEMV that follows: no reconfiguration of the SMs between the two
        cudaFuncSetAttribute(quantize_absmax_int8_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
        configured[dev] = true;
    }
    quantize_absmax_int8_kernel<<<1, kQuantThreads, smem, stream>>>(x, q, scale, n);
    return check_launch("quantize_absmax_int8");
}

}  // namespace tllm
