// The operators either side of the ternary contraction inside a decoder layer:
// RMSNorm (with residual add and, for the INT8 decode path, the absmax quantiser fused
// in), rotary embedding fused with the KV-cache append, SwiGLU (optionally with the
// quantiser), residual add, embedding lookup, the FP16 lm_head GEMV, FP16 GEMM and a
// device-side argmax.  Semantics follow the reference operators declared in its
// include/kernels.cuh:45-86 (kernels/rmsnorm.cu, rope.cu, activations.cu,
// elementwise.cu); the kernels are written for B200: 128-bit accesses, one pass over
// global memory with the working vector staged in shared memory, programmatic dependent
// launch, and positions / scales read from device memory so that a whole decode step
// replays as one CUDA graph without a host round trip.
#include <cfloat>

#include "launch.cuh"
#include "layer.cuh"

namespace tllm {

constexpr int kNormThreads = 512;

__device__ __forceinline__ float block_sum(float v, float* sh)
{
    v = warp_sum(v);
    const int tid = threadIdx.x;
    __syncthreads();
    if ((tid & 31) == 0) sh[tid >> 5] = v;
    __syncthreads();
    float t = (tid < (int)(blockDim.x >> 5)) ? sh[tid] : 0.f;
    if (tid < 32) {
        t = warp_sum(t);
        if (tid == 0) sh[0] = t;
    }
    __syncthreads();
    return sh[0];
}

__device__ __forceinline__ float block_max(float v, float* sh)
{
    v = warp_max(v);
    const int tid = threadIdx.x;
    __syncthreads();
    if ((tid & 31) == 0) sh[tid >> 5] = v;
    __syncthreads();
    float t = (tid < (int)(blockDim.x >> 5)) ? sh[tid] : -FLT_MAX;
    if (tid < 32) {
        t = warp_max(t);
        if (tid == 0) sh[0] = t;
    }
    __syncthreads();
    return sh[0];
}

// absmax quantisation of `n` staged floats (each already rounded to FP16), semantics of
// the reference quantiser (kernels/activations.cu:88-142): scale = absmax / 127, or 1
// for an all-zero vector; q = clamp(rint(x * (127 / absmax)), -127, 127).
__device__ __forceinline__ void quantize_staged(const float* vals, int n, int8_t* q, float* scale_out, float* sh)
{
    float m = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, fabsf(vals[i]));
    const float absmax = block_max(m, sh);
    if (threadIdx.x == 0) *scale_out = (absmax > 0.f) ? (absmax / 127.0f) : 1.0f;
    const float inv = (absmax > 0.f) ? (127.0f / absmax) : 0.f;
    if ((n & 3) == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0) {
        for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(vals + 4 * i);
            const int q0 = max(-127, min(127, __float2int_rn(v.x * inv))), q1 = max(-127, min(127, __float2int_rn(v.y * inv)));
            const int q2 = max(-127, min(127, __float2int_rn(v.z * inv))), q3 = max(-127, min(127, __float2int_rn(v.w * inv)));
            reinterpret_cast<uint32_t*>(q)[i] = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) |
                                                ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
        }
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x)
            q[i] = (int8_t)max(-127, min(127, __float2int_rn(vals[i] * inv)));
    }
}

// ---------------------------------------------------------------------------
// RMSNorm (+ residual add) (+ INT8 quantisation)      reference: kernels/rmsnorm.cu:19-103
// ---------------------------------------------------------------------------
// One CTA per token (output pointers may alias inputs: every element is read and written
// by the same thread).  tmp = input (+ residual); residual_out = half(tmp);
// var = sum(tmp^2) / dim (of the unrounded sum, as the reference computes it);
// output = half(v * rsqrt(var + eps) * weight) with v = the rounded residual_out when it
// was stored, else tmp.  With q != nullptr the normalised vector is also quantised.
// round_first: var is taken over the rounded sum, which is what the reference engine's
// add_forward followed by rmsnorm_forward computes (src/transformer.cpp:252-261).
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(const half* __restrict__ input, const half* __restrict__ weight, half* __restrict__ output,
               const half* residual, half* residual_out, int8_t* __restrict__ q,
               float* __restrict__ q_scale, int dim, float eps, int round_first)
{
    extern __shared__ __align__(16) float vals[];      // [dim]
    __shared__ float sh[32];
    pdl_launch_dependents();
    const int tid = threadIdx.x;
    const size_t base = (size_t)blockIdx.x * dim;
    pdl_wait();

    const half* xin = input + base;
    const half* rin = residual ? residual + base : nullptr;
    half* rout = residual_out ? residual_out + base : nullptr;
    half* yout = output + base;
    const bool vec = ((dim & 7) == 0) && (((reinterpret_cast<uintptr_t>(xin) | reinterpret_cast<uintptr_t>(rin) |
                                            reinterpret_cast<uintptr_t>(rout) | reinterpret_cast<uintptr_t>(yout) |
                                            reinterpret_cast<uintptr_t>(weight)) & 15) == 0);
    // element-wise part of the first pass; returns the value kept for the second pass
    auto first = [&](float x, float r, bool has_r, half& stored, float& ss) -> float {
        float v = x;
        if (has_r) {
            v += r;
            if (!round_first) ss += v * v;
            if (rout) {
                stored = __float2half_rn(v);
                v = __half2float(stored);
            }
            if (round_first) ss += v * v;
        } else {
            ss += v * v;
        }
        return v;
    };
    float ss = 0.f;
    if (vec) {
        for (int i = tid; i < dim / 8; i += kNormThreads) {
            const uint4 xr = *(reinterpret_cast<const uint4*>(xin) + i);
            uint4 rr = make_uint4(0, 0, 0, 0);
            if (rin) rr = *(reinterpret_cast<const uint4*>(rin) + i);
            const half* xh = reinterpret_cast<const half*>(&xr);
            const half* rh = reinterpret_cast<const half*>(&rr);
            uint4 st4;
            half* sth = reinterpret_cast<half*>(&st4);
#pragma unroll
            for (int j = 0; j < 8; j++)
                vals[i * 8 + j] = first(__half2float(xh[j]), __half2float(rh[j]), rin != nullptr, sth[j], ss);
            if (rin && rout) *(reinterpret_cast<uint4*>(rout) + i) = st4;
        }
    } else {
        for (int i = tid; i < dim; i += kNormThreads) {
            half stored;
            vals[i] = first(__half2float(xin[i]), rin ? __half2float(rin[i]) : 0.f, rin != nullptr, stored, ss);
            if (rin && rout) rout[i] = stored;
        }
    }
    const float var = block_sum(ss, sh) / (float)dim;
    const float rinv = rsqrtf(var + eps);
    if (vec) {
        for (int i = tid; i < dim / 8; i += kNormThreads) {
            const uint4 wr = __ldg(reinterpret_cast<const uint4*>(weight) + i);
            const half* wh = reinterpret_cast<const half*>(&wr);
            uint4 st4;
            half* sth = reinterpret_cast<half*>(&st4);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                sth[j] = __float2half_rn(vals[i * 8 + j] * rinv * __half2float(wh[j]));
                vals[i * 8 + j] = __half2float(sth[j]);
            }
            *(reinterpret_cast<uint4*>(yout) + i) = st4;
        }
    } else {
        for (int i = tid; i < dim; i += kNormThreads) {
            const half o = __float2half_rn(vals[i] * rinv * __half2float(weight[i]));
            yout[i] = o;
            vals[i] = __half2float(o);
        }
    }
    if (q) {
        __syncthreads();
        quantize_staged(vals, dim, q + base, q_scale + blockIdx.x, sh);
    }
}

int launch_rmsnorm(const half* input, const half* weight, half* output, const half* residual, half* residual_out,
                   int8_t* q, float* q_scale, int batch, int dim, float eps, int round_first, cudaStream_t stream)
{
    if (batch == 0) return TLLM_OK;
    const size_t smem = (size_t)dim * sizeof(float);
    if (smem > 200 * 1024) return fail(TLLM_ERR_SHAPE, "rmsnorm: dim=%d exceeds %d", dim, 200 * 1024 / 4);
    static bool attr[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr[dev]) {
        cudaFuncSetAttribute(rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr[dev] = true;
    }
    return launch_pdl("rmsnorm", rmsnorm_kernel, dim3(batch), dim3(kNormThreads), smem, stream, input, weight, output,
                      residual, residual_out, q, q_scale, dim, eps, round_first);
}

// ---------------------------------------------------------------------------
// Rotary embedding, optionally fused with the KV-cache append
//   reference: kernels/rope.cu:21-78 (interleaved pairs (2i, 2i+1), angle =
//   pos / theta^(2i/head_dim)), kernels/elementwise.cu:97-128 (cache layout
//   [batch, n_kv_heads, max_seq_len, head_dim], positions beyond the cache dropped)
// ---------------------------------------------------------------------------
// One thread per (batch, token, head, pair).  q and k are rotated in place; when caches
// are given the rotated k pair and the v pair of kv heads go to cache position
// start_pos + token.  start_pos comes from device memory when pos_dev != nullptr.
__global__ void __launch_bounds__(256)
rope_kernel(half* __restrict__ q, half* __restrict__ k, const half* __restrict__ v, half* __restrict__ k_cache,
            half* __restrict__ v_cache, int batch, int seq_len, int n_heads, int n_kv_heads, int head_dim,
            int start_pos, const int* __restrict__ pos_dev, float theta, int max_seq_len, int do_rope)
{
    pdl_launch_dependents();
    const int half_dim = head_dim >> 1;
    const int max_heads = max(n_heads, n_kv_heads);
    const long long total = (long long)batch * seq_len * max_heads * half_dim;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int pair = (int)(idx % half_dim);
    long long t = idx / half_dim;
    const int head = (int)(t % max_heads);
    t /= max_heads;
    const int s = (int)(t % seq_len);
    const int b = (int)(t / seq_len);
    const float freq = 1.0f / powf(theta, (2.0f * (float)pair) / (float)head_dim);
    pdl_wait();
    if (pos_dev) start_pos = *pos_dev;
    const int pos = start_pos + s;
    float sn = 0.f, cs = 1.f;
    if (do_rope) sincosf((float)pos * freq, &sn, &cs);

    if (head < n_heads && do_rope) {
        half2* p = reinterpret_cast<half2*>(q + (((size_t)b * seq_len + s) * n_heads + head) * head_dim) + pair;
        const float2 x = __half22float2(*p);
        *p = __halves2half2(__float2half_rn(x.x * cs - x.y * sn), __float2half_rn(x.x * sn + x.y * cs));
    }
    if (head < n_kv_heads) {
        const size_t src = (((size_t)b * seq_len + s) * n_kv_heads + head) * head_dim;
        half2 kr = *(reinterpret_cast<const half2*>(k + src) + pair);
        if (do_rope) {
            const float2 x = __half22float2(kr);
            kr = __halves2half2(__float2half_rn(x.x * cs - x.y * sn), __float2half_rn(x.x * sn + x.y * cs));
            *(reinterpret_cast<half2*>(k + src) + pair) = kr;
        }
        if (k_cache && pos < max_seq_len) {
            const size_t dst = (((size_t)b * n_kv_heads + head) * max_seq_len + pos) * head_dim;
            *(reinterpret_cast<half2*>(k_cache + dst) + pair) = kr;
            *(reinterpret_cast<half2*>(v_cache + dst) + pair) = *(reinterpret_cast<const half2*>(v + src) + pair);
        }
    }
}

int launch_rope(half* q, half* k, const half* v, half* k_cache, half* v_cache, int batch, int seq_len, int n_heads,
                int n_kv_heads, int head_dim, int start_pos, const int* pos_dev, float theta, int max_seq_len,
                int do_rope, cudaStream_t stream)
{
    const int max_heads = n_heads > n_kv_heads ? n_heads : n_kv_heads;
    const long long total = (long long)batch * seq_len * max_heads * (head_dim / 2);
    if (total == 0) return TLLM_OK;
    const unsigned grid = (unsigned)((total + 255) / 256);
    return launch_pdl("rope", rope_kernel, dim3(grid), dim3(256), 0, stream, q, k, v, k_cache, v_cache, batch, seq_len,
                      n_heads, n_kv_heads, head_dim, start_pos, pos_dev, theta, max_seq_len, do_rope);
}

// ---------------------------------------------------------------------------
// SwiGLU   out = half(g / (1 + exp(-g)) * u)       reference: kernels/activations.cu:18-74
// ---------------------------------------------------------------------------
__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }

__global__ void __launch_bounds__(256)
silu_mul_kernel(const half* gate, const half* up, half* out, long long size)
{
    pdl_launch_dependents();
    const long long i2 = (long long)blockIdx.x * blockDim.x + threadIdx.x;     // pair index
    pdl_wait();
    if (2 * i2 + 1 < size) {
        const float2 g = __half22float2(reinterpret_cast<const half2*>(gate)[i2]);
        const float2 u = __half22float2(reinterpret_cast<const half2*>(up)[i2]);
        reinterpret_cast<half2*>(out)[i2] =
            __halves2half2(__float2half_rn(silu_mul(g.x, u.x)), __float2half_rn(silu_mul(g.y, u.y)));
    } else if (2 * i2 < size) {
        out[2 * i2] = __float2half_rn(silu_mul(__half2float(gate[2 * i2]), __half2float(up[2 * i2])));
    }
}

// Decode form: one vector, SwiGLU and the absmax quantiser in one CTA (the quantiser
// needs the maximum over the whole vector before it can write a byte).
__global__ void __launch_bounds__(1024)
silu_mul_quant_kernel(const half* gate, const half* up, half* out, int8_t* __restrict__ q,
                      float* __restrict__ q_scale, int size)
{
    extern __shared__ __align__(16) float vals[];
    __shared__ float sh[32];
    pdl_launch_dependents();
    pdl_wait();
    if ((size & 7) == 0 && ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) |
                             reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        for (int i = threadIdx.x; i < size / 8; i += blockDim.x) {
            const uint4 gr = *(reinterpret_cast<const uint4*>(gate) + i);
            const uint4 ur = *(reinterpret_cast<const uint4*>(up) + i);
            const half* gh = reinterpret_cast<const half*>(&gr);
            const half* uh = reinterpret_cast<const half*>(&ur);
            uint4 st4;
            half* sth = reinterpret_cast<half*>(&st4);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                sth[j] = __float2half_rn(silu_mul(__half2float(gh[j]), __half2float(uh[j])));
                vals[i * 8 + j] = __half2float(sth[j]);
            }
            *(reinterpret_cast<uint4*>(out) + i) = st4;
        }
    } else {
        for (int i = threadIdx.x; i < size; i += blockDim.x) {
            const half o = __float2half_rn(silu_mul(__half2float(gate[i]), __half2float(up[i])));
            out[i] = o;
            vals[i] = __half2float(o);
        }
    }
    __syncthreads();
    quantize_staged(vals, size, q, q_scale, sh);
}

int launch_silu_mul(const half* gate, const half* up, half* out, long long size, int8_t* q, float* q_scale,
                    cudaStream_t stream)
{
    if (size == 0) return TLLM_OK;
    if (q) {
        const size_t smem = (size_t)size * sizeof(float);
        if (smem > 200 * 1024) return fail(TLLM_ERR_SHAPE, "silu_mul+quantise: size=%lld exceeds %d", size, 200 * 1024 / 4);
        static bool attr[64] = {};
        int dev = 0;
        cudaGetDevice(&dev);
        if (!attr[dev]) {
            cudaFuncSetAttribute(silu_mul_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            attr[dev] = true;
        }
        return launch_pdl("silu_mul_quant", silu_mul_quant_kernel, dim3(1), dim3(1024), smem, stream, gate, up, out, q,
                          q_scale, (int)size);
    }
    const long long pairs = (size + 1) / 2;
    return launch_pdl("silu_mul", silu_mul_kernel, dim3((unsigned)((pairs + 255) / 256)), dim3(256), 0, stream, gate,
                      up, out, size);
}

// ---------------------------------------------------------------------------
// Residual add   out = half(float(a) + float(b))     reference: kernels/elementwise.cu:19-49
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
add_kernel(const half* a, const half* b, half* out, long long size)
{
    pdl_launch_dependents();
    const long long i2 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    pdl_wait();
    if (2 * i2 + 1 < size) {
        const float2 x = __half22float2(reinterpret_cast<const half2*>(a)[i2]);
        const float2 y = __half22float2(reinterpret_cast<const half2*>(b)[i2]);
        reinterpret_cast<half2*>(out)[i2] = __halves2half2(__float2half_rn(x.x + y.x), __float2half_rn(x.y + y.y));
    } else if (2 * i2 < size) {
        out[2 * i2] = __float2half_rn(__half2float(a[2 * i2]) + __half2float(b[2 * i2]));
    }
}

int launch_add(const half* a, const half* b, half* out, long long size, cudaStream_t stream)
{
    if (size == 0) return TLLM_OK;
    const long long pairs = (size + 1) / 2;
    return launch_pdl("add", add_kernel, dim3((unsigned)((pairs + 255) / 256)), dim3(256), 0, stream, a, b, out, size);
}

// ---------------------------------------------------------------------------
// Embedding lookup   out[t, :] = table[indices[t], :]     reference: kernels/elementwise.cu:55-88
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
embedding_kernel(const half* __restrict__ table, const int* __restrict__ indices, half* __restrict__ out, int dim)
{
    pdl_launch_dependents();
    pdl_wait();
    const half* src = table + (size_t)indices[blockIdx.x] * dim;
    half* dst = out + (size_t)blockIdx.x * dim;
    if ((dim & 7) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
        for (int i = threadIdx.x; i < dim / 8; i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] = __ldg(reinterpret_cast<const uint4*>(src) + i);
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = src[i];
    }
}

int launch_embedding(const half* table, const int* indices, half* out, int n_tokens, int dim, cudaStream_t stream)
{
    if (n_tokens == 0) return TLLM_OK;
    return launch_pdl("embedding", embedding_kernel, dim3(n_tokens), dim3(256), 0, stream, table, indices, out, dim);
}

// ---------------------------------------------------------------------------
// FP16 GEMV   y[r] = half(sum_c float(W[r, c]) * float(x[c]))    reference: kernels/elementwise.cu:158-201
// ---------------------------------------------------------------------------
// The lm_head of the 1B configuration is 525 MB of FP16, twice the ternary bytes of the
// whole layer stack, so this kernel is HBM-bound like the ternary GEMV: x is staged in
// shared memory once per CTA, each warp streams whole rows with 128-bit loads, four
// loads in flight per lane, FP32 accumulation.
constexpr int kFp16GemvWarps = 8;

__global__ void __launch_bounds__(kFp16GemvWarps * 32)
fp16_gemv_kernel(const half* __restrict__ w, const half* __restrict__ x, half* __restrict__ y, int rows, int cols)
{
    extern __shared__ __align__(16) half xs[];
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_wait();
    for (int i = threadIdx.x; i < cols; i += blockDim.x) xs[i] = x[i];
    __syncthreads();
    const bool vec = ((cols & 7) == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    for (int r = blockIdx.x * kFp16GemvWarps + warp; r < rows; r += gridDim.x * kFp16GemvWarps) {
        const half* wr = w + (size_t)r * cols;
        float acc = 0.f;
        if (vec) {
            const uint4* w4 = reinterpret_cast<const uint4*>(wr);
            const uint4* x4 = reinterpret_cast<const uint4*>(xs);
            const int n8 = cols >> 3;
            int c = lane;
            for (; c + 96 < n8; c += 128) {
                uint4 a[4];
#pragma unroll
                for (int u = 0; u < 4; u++) a[u] = __ldcs(w4 + c + 32 * u);
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const uint4 b = x4[c + 32 * u];
                    const half2* ah = reinterpret_cast<const half2*>(&a[u]);
                    const half2* bh = reinterpret_cast<const half2*>(&b);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float2 fa = __half22float2(ah[j]), fb = __half22float2(bh[j]);
                        acc = fmaf(fa.x, fb.x, acc);
                        acc = fmaf(fa.y, fb.y, acc);
                    }
                }
            }
            for (; c < n8; c += 32) {
                const uint4 a = __ldcs(w4 + c), b = x4[c];
                const half2* ah = reinterpret_cast<const half2*>(&a);
                const half2* bh = reinterpret_cast<const half2*>(&b);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 fa = __half22float2(ah[j]), fb = __half22float2(bh[j]);
                    acc = fmaf(fa.x, fb.x, acc);
                    acc = fmaf(fa.y, fb.y, acc);
                }
            }
        } else {
            for (int c = lane; c < cols; c += 32) acc = fmaf(__half2float(wr[c]), __half2float(xs[c]), acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) y[r] = __float2half_rn(acc);
    }
}

int launch_fp16_gemv(const half* w, const half* x, half* y, int rows, int cols, cudaStream_t stream)
{
    if (rows == 0) return TLLM_OK;
    const size_t smem = (size_t)cols * sizeof(half);
    if (smem > 200 * 1024) return fail(TLLM_ERR_SHAPE, "fp16_gemv: cols=%d exceeds %d", cols, 100 * 1024);
    static bool attr[64] = {};
    static int sms[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr[dev]) {
        cudaFuncSetAttribute(fp16_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
        attr[dev] = true;
    }
    long long grid = ((long long)rows + kFp16GemvWarps - 1) / kFp16GemvWarps;
    const long long cap = (long long)sms[dev] * 8;
    if (grid > cap) grid = cap;
    return launch_pdl("fp16_gemv", fp16_gemv_kernel, dim3((unsigned)grid), dim3(kFp16GemvWarps * 32), smem, stream, w, x,
                      y, rows, cols);
}

// Several vectors at once (batched decode): y[b, r] = W[r, :] . x[b, :].  The vectors are taken
// eight at a time: staged in shared memory, every weight row read once per eight vectors.
constexpr int kFp16GemvVecs = 8;

__global__ void __launch_bounds__(kFp16GemvWarps * 32)
fp16_gemv_batched_kernel(const half* __restrict__ w, const half* __restrict__ x, half* __restrict__ y, int batch,
                         int rows, int cols)
{
    extern __shared__ __align__(16) half xs[];          // [kFp16GemvVecs][cols]
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_wait();
    for (int b0 = 0; b0 < batch; b0 += kFp16GemvVecs) {
        const int nb = min(kFp16GemvVecs, batch - b0);
        __syncthreads();
        for (int i = threadIdx.x; i < nb * cols; i += blockDim.x) xs[i] = x[(size_t)b0 * cols + i];
        __syncthreads();
        for (int r = blockIdx.x * kFp16GemvWarps + warp; r < rows; r += gridDim.x * kFp16GemvWarps) {
            const half* wr = w + (size_t)r * cols;
            float acc[kFp16GemvVecs];
#pragma unroll
            for (int b = 0; b < kFp16GemvVecs; b++) acc[b] = 0.f;
            if ((cols & 7) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
                for (int c = lane; c < (cols >> 3); c += 32) {
                    const uint4 a = __ldcs(reinterpret_cast<const uint4*>(wr) + c);
                    const half2* ah = reinterpret_cast<const half2*>(&a);
                    float2 fa[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) fa[j] = __half22float2(ah[j]);
#pragma unroll
                    for (int b = 0; b < kFp16GemvVecs; b++) {
                        if (b < nb) {
                            const uint4 xv = *(reinterpret_cast<const uint4*>(xs + (size_t)b * cols) + c);
                            const half2* xh = reinterpret_cast<const half2*>(&xv);
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                const float2 fx = __half22float2(xh[j]);
                                acc[b] = fmaf(fa[j].x, fx.x, acc[b]);
                                acc[b] = fmaf(fa[j].y, fx.y, acc[b]);
                            }
                        }
                    }
                }
            } else {
                for (int c = lane; c < cols; c += 32) {
                    const float fw = __half2float(wr[c]);
#pragma unroll
                    for (int b = 0; b < kFp16GemvVecs; b++)
                        if (b < nb) acc[b] = fmaf(fw, __half2float(xs[(size_t)b * cols + c]), acc[b]);
                }
            }
#pragma unroll
            for (int b = 0; b < kFp16GemvVecs; b++) {
                if (b < nb) {
                    const float v = warp_sum(acc[b]);
                    if (lane == 0) y[(size_t)(b0 + b) * rows + r] = __float2half_rn(v);
                }
            }
        }
    }
}

int launch_fp16_gemv_batched(const half* w, const half* x, half* y, int batch, int rows, int cols, cudaStream_t stream)
{
    if (rows == 0 || batch == 0) return TLLM_OK;
    if (batch == 1) return launch_fp16_gemv(w, x, y, rows, cols, stream);
    const size_t smem = (size_t)kFp16GemvVecs * cols * sizeof(half);
    if (smem > 200 * 1024) return fail(TLLM_ERR_SHAPE, "fp16_gemv (batched): cols=%d exceeds %d", cols, 200 * 1024 / 16);
    static bool attr[64] = {};
    static int sms[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr[dev]) {
        cudaFuncSetAttribute(fp16_gemv_batched_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
        attr[dev] = true;
    }
    long long grid = ((long long)rows + kFp16GemvWarps - 1) / kFp16GemvWarps;
    const long long cap = (long long)sms[dev] * 4;
    if (grid > cap) grid = cap;
    return launch_pdl("fp16_gemv_batched", fp16_gemv_batched_kernel, dim3((unsigned)grid), dim3(kFp16GemvWarps * 32), smem,
                      stream, w, x, y, batch, rows, cols);
}

// ---------------------------------------------------------------------------
// FP16 GEMM   C[M, N] = A[M, K] . B[N, K]^T, FP32 accumulation   reference: kernels/elementwise.cu:216-304
// ---------------------------------------------------------------------------
// Off the decode path (the engine calls it only for an FP16 lm_head over several tokens,
// which its forward pass never requests).  C[M,N] = A[M,K] . B[N,K]^T on mma.sync.m16n8k16:
// A is row-major along K and B[N,K] is exactly the "col" operand, so every lane loads its
// operand fragments straight from global memory as 32-bit words (two consecutive K values of
// one row) -- no shared memory, no transposition.  A CTA of four warps owns 64 x 64 of C, a
// warp 32 x 32 (2 x 4 MMA tiles, FP32 accumulators).  Edges and odd K go through guarded
// element loads.
__device__ __forceinline__ uint32_t gemm_pair(const half* __restrict__ p, int row, int rows, int k, int K, bool vec)
{
    if (row >= rows) return 0u;
    const half* q = p + (size_t)row * K + k;
    if (vec && k + 1 < K) return __ldg(reinterpret_cast<const unsigned int*>(q));
    const unsigned short lo = (k < K) ? __half_as_ushort(q[0]) : (unsigned short)0;
    const unsigned short hi = (k + 1 < K) ? __half_as_ushort(q[1]) : (unsigned short)0;
    return (uint32_t)lo | ((uint32_t)hi << 16);
}

__global__ void __launch_bounds__(128)
fp16_gemm_kernel(const half* __restrict__ A, const half* __restrict__ B, half* __restrict__ C, int M, int N, int K)
{
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gq = lane >> 2, t = lane & 3;
    const int m0 = blockIdx.y * 64 + (warp >> 1) * 32, n0 = blockIdx.x * 64 + (warp & 1) * 32;
    // 32-bit loads need an even K (rows then start on 4-byte boundaries) and aligned bases
    const bool vec = (K & 1) == 0 && ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 3) == 0;
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[i][j][e] = 0.f;
    pdl_wait();
    for (int k0 = 0; k0 < K; k0 += 16) {
        uint32_t a[2][4], b[4][2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int r = m0 + i * 16 + gq;
            a[i][0] = gemm_pair(A, r, M, k0 + 2 * t, K, vec);
            a[i][1] = gemm_pair(A, r + 8, M, k0 + 2 * t, K, vec);
            a[i][2] = gemm_pair(A, r, M, k0 + 2 * t + 8, K, vec);
            a[i][3] = gemm_pair(A, r + 8, M, k0 + 2 * t + 8, K, vec);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int c = n0 + j * 8 + gq;
            b[j][0] = gemm_pair(B, c, N, k0 + 2 * t, K, vec);
            b[j][1] = gemm_pair(B, c, N, k0 + 2 * t + 8, K, vec);
        }
#pragma unroll
        for (int i = 0; i < 2; i++)
#pragma unroll
            for (int j = 0; j < 4; j++)
                asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                    : "+f"(acc[i][j][0]), "+f"(acc[i][j][1]), "+f"(acc[i][j][2]), "+f"(acc[i][j][3])
                    : "r"(a[i][0]), "r"(a[i][1]), "r"(a[i][2]), "r"(a[i][3]), "r"(b[j][0]), "r"(b[j][1]));
    }
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int m = m0 + i * 16 + gq + (e >> 1) * 8, n = n0 + j * 8 + 2 * t + (e & 1);
                if (m < M && n < N) C[(size_t)m * N + n] = __float2half_rn(acc[i][j][e]);
            }
}

int launch_fp16_gemm(const half* A, const half* B, half* C, int M, int N, int K, cudaStream_t stream)
{
    if (M == 0 || N == 0) return TLLM_OK;
    return launch_pdl("fp16_gemm", fp16_gemm_kernel, dim3((N + 63) / 64, (M + 63) / 64), dim3(128), 0, stream, A, B, C,
                      M, N, K);
}

// ---------------------------------------------------------------------------
// Greedy sampling on the device: index of the largest logit (lowest index on ties)
// ---------------------------------------------------------------------------
// Two levels in one launch: every CTA reduces a slice, the CTA that arrives last (a
// counter that it resets, so that graph replays start clean) reduces the slices and
// writes the token to `out` and, when given, to `history[*step]`, then advances *step.
constexpr int kArgmaxCtas = 64;
constexpr int kArgmaxThreads = 256;

__global__ void __launch_bounds__(kArgmaxThreads)
argmax_kernel(const half* __restrict__ logits, int n, int* __restrict__ out, int* __restrict__ history,
              int* __restrict__ step, float* __restrict__ part_val, int* __restrict__ part_idx,
              unsigned* __restrict__ counter, int* __restrict__ pos)
{
    __shared__ float sv[kArgmaxThreads / 32];
    __shared__ int si[kArgmaxThreads / 32];
    __shared__ int s_last;
    pdl_launch_dependents();
    pdl_wait();
    float best = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int i = blockIdx.x * kArgmaxThreads + threadIdx.x; i < n; i += kArgmaxCtas * kArgmaxThreads) {
        const float v = __half2float(logits[i]);
        if (v > best || (v == best && i < bi)) {
            best = v;
            bi = i;
        }
    }
    auto reduce = [&](float& v, int& idx) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > v || (ov == v && oi < idx)) {
                v = ov;
                idx = oi;
            }
        }
    };
    reduce(best, bi);
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = best;
        si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = (threadIdx.x < kArgmaxThreads / 32) ? sv[threadIdx.x] : -FLT_MAX;
        int idx = (threadIdx.x < kArgmaxThreads / 32) ? si[threadIdx.x] : 0x7fffffff;
        reduce(v, idx);
        if (threadIdx.x == 0) {
            part_val[blockIdx.x] = v;
            part_idx[blockIdx.x] = idx;
            __threadfence();
            s_last = (atomicAdd(counter, 1u) == kArgmaxCtas - 1) ? 1 : 0;
        }
    }
    __syncthreads();
    if (!s_last || threadIdx.x >= 32) return;
    __threadfence();
    float v = -FLT_MAX;
    int idx = 0x7fffffff;
    for (int c = threadIdx.x; c < kArgmaxCtas; c += 32) {
        const float ov = __ldcg(part_val + c);
        const int oi = __ldcg(part_idx + c);
        if (ov > v || (ov == v && oi < idx)) {
            v = ov;
            idx = oi;
        }
    }
    reduce(v, idx);
    if (threadIdx.x == 0) {
        if (idx == 0x7fffffff) idx = 0;
        *out = idx;
        if (history && step) {
            history[*step] = idx;
            *step = *step + 1;
        }
        if (pos) *pos = *pos + 1;      // the decode loop's cache position moves on with the token
        *counter = 0;
    }
}

int launch_argmax(const half* logits, int n, int* out, int* history, int* step, float* part_val, int* part_idx,
                  unsigned* counter, int* pos, cudaStream_t stream)
{
    return launch_pdl("argmax", argmax_kernel, dim3(kArgmaxCtas), dim3(kArgmaxThreads), 0, stream, logits, n, out,
                      history, step, part_val, part_idx, counter, pos);
}

}  // namespace tllm

