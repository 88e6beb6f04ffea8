// General-shape ternary GEMV on the reference layout, CUDA cores only.
//
// This is the path for shapes the tensor-core streaming kernels do not take
// (rows not a multiple of 16) and the plain restatement every other kernel is
// compared with in the tests.  One warp owns one output row; each lane takes
// whole scale groups (one 128-bit load of nonzero bits, one of sign bits, one
// scale), so a warp-wide load covers 32 consecutive groups of the row.  The
// select is branch-free: t = nz_bit * (2*sign_bit - 1).
//
// Semantics follow the reference kernels/ternary_gemv.cu:27-87 (FP16 input) and
// :116-199 (INT8 input): FP32 (resp. exact INT32) group sums, scale applied once
// per group, FP32 row sum, FP16 store.
#include "common.cuh"

namespace tllm {

constexpr int kSimtWarps = 8;

template <int B>
__global__ void __launch_bounds__(kSimtWarps * 32)
gemv_simt_kernel(const uint4* __restrict__ nz, const uint4* __restrict__ sg,
                 const half* __restrict__ scales, const half* __restrict__ x,
                 half* __restrict__ y, int rows, int cols)
{
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * kSimtWarps + (threadIdx.x >> 5);
    if (row >= rows) return;                      // whole warps leave; no barrier follows
    const int groups = cols / kGroup;
    const uint4* nzr = nz + (size_t)row * groups;
    const uint4* sgr = sg + (size_t)row * groups;
    const half* sr = scales + (size_t)row * groups;

    float acc[B];
#pragma unroll
    for (int b = 0; b < B; b++) acc[b] = 0.f;

    for (int g = lane; g < groups; g += 32) {
        const uint4 a4 = __ldg(nzr + g);
        const uint4 s4 = __ldg(sgr + g);
        const float sc = __half2float(__ldg(sr + g));
        const uint32_t aw[4] = {a4.x, a4.y, a4.z, a4.w};
        const uint32_t sw[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int b = 0; b < B; b++) {
            const uint4* xg = reinterpret_cast<const uint4*>(x + (size_t)b * cols + (size_t)g * kGroup);
            float gsum = 0.f;
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const uint32_t pos = aw[w] & sw[w], neg = aw[w] & ~sw[w];
#pragma unroll
                for (int q = 0; q < 4; q++) {     // 8 activations per 128-bit load
                    const uint4 xv = __ldg(xg + w * 4 + q);
                    const uint32_t xr[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                    for (int p = 0; p < 4; p++) {
                        const float2 f = __half22float2(*reinterpret_cast<const half2*>(&xr[p]));
                        const int bit = q * 8 + p * 2;
                        const float t0 = (float)((int)((pos >> bit) & 1u) - (int)((neg >> bit) & 1u));
                        const float t1 = (float)((int)((pos >> (bit + 1)) & 1u) - (int)((neg >> (bit + 1)) & 1u));
                        gsum = fmaf(t0, f.x, gsum);
                        gsum = fmaf(t1, f.y, gsum);
                    }
                }
            }
            acc[b] = fmaf(sc, gsum, acc[b]);
        }
    }
#pragma unroll
    for (int b = 0; b < B; b++) {
        const float v = warp_sum(acc[b]);
        if (lane == 0) y[(size_t)b * rows + row] = __float2half_rn(v);
    }
}

__global__ void __launch_bounds__(kSimtWarps * 32)
gemv_int8_simt_kernel(const uint4* __restrict__ nz, const uint4* __restrict__ sg,
                      const half* __restrict__ scales, const int8_t* __restrict__ xq,
                      float input_scale, half* __restrict__ y, int rows, int cols)
{
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * kSimtWarps + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int groups = cols / kGroup;
    const uint4* nzr = nz + (size_t)row * groups;
    const uint4* sgr = sg + (size_t)row * groups;
    const half* sr = scales + (size_t)row * groups;

    float acc = 0.f;
    for (int g = lane; g < groups; g += 32) {
        const uint4 a4 = __ldg(nzr + g);
        const uint4 s4 = __ldg(sgr + g);
        const float sc = __half2float(__ldg(sr + g));
        const uint32_t aw[4] = {a4.x, a4.y, a4.z, a4.w};
        const uint32_t sw[4] = {s4.x, s4.y, s4.z, s4.w};
        const uint4* xg = reinterpret_cast<const uint4*>(xq + (size_t)g * kGroup);
        int gsum = 0;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const uint32_t pos = aw[w] & sw[w], neg = aw[w] & ~sw[w];
#pragma unroll
            for (int q = 0; q < 2; q++) {         // 16 activations per 128-bit load
                const uint4 xv = __ldg(xg + w * 2 + q);
                const uint32_t xr[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int p = 0; p < 4; p++) {
                    const int bit = q * 16 + p * 4;
                    uint32_t wp = 0;              // four ternary weights as int8 lanes
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const int t = (int)((pos >> (bit + j)) & 1u) - (int)((neg >> (bit + j)) & 1u);
                        wp |= (uint32_t)(t & 0xff) << (8 * j);
                    }
                    gsum = __dp4a((int)wp, (int)xr[p], gsum);
                }
            }
        }
        acc = fmaf(sc, (float)gsum, acc);
    }
    acc = warp_sum(acc) * input_scale;
    if (lane == 0) y[row] = __float2half_rn(acc);
}

template <int B>
static int launch_b(const uint32_t* nz, const uint32_t* sg, const half* scales, const half* x,
                    half* y, int rows, int cols, cudaStream_t stream)
{
    const int grid = (rows + kSimtWarps - 1) / kSimtWarps;
    gemv_simt_kernel<B><<<grid, kSimtWarps * 32, 0, stream>>>(
        reinterpret_cast<const uint4*>(nz), reinterpret_cast<const uint4*>(sg), scales, x, y, rows, cols);
    return check_launch("gemv_simt");
}

int launch_gemv_simt(const uint32_t* nz, const uint32_t* sg, const half* scales, const half* x,
                     half* y, int batch, int rows, int cols, cudaStream_t stream)
{
    // Register use grows with the batch held per pass; larger batches run as
    // passes of at most 4 vectors.
    int done = 0;
    while (done < batch) {
        const int b = (batch - done >= 4) ? 4 : (batch - done);
        const half* xb = x + (size_t)done * cols;
        half* yb = y + (size_t)done * rows;
        int st;
        switch (b) {
            case 4: st = launch_b<4>(nz, sg, scales, xb, yb, rows, cols, stream); break;
            case 3: st = launch_b<3>(nz, sg, scales, xb, yb, rows, cols, stream); break;
            case 2: st = launch_b<2>(nz, sg, scales, xb, yb, rows, cols, stream); break;
            default: st = launch_b<1>(nz, sg, scales, xb, yb, rows, cols, stream); break;
        }
        if (st != TLLM_OK) return st;
        done += b;
    }
    return TLLM_OK;
}

int launch_gemv_int8_simt(const uint32_t* nz, const uint32_t* sg, const half* scales,
                          const int8_t* xq, float input_scale, half* y, int rows, int cols,
                          cudaStream_t stream)
{
    const int grid = (rows + kSimtWarps - 1) / kSimtWarps;
    gemv_int8_simt_kernel<<<grid, kSimtWarps * 32, 0, stream>>>(
        reinterpret_cast<const uint4*>(nz), reinterpret_cast<const uint4*>(sg), scales, xq,
        input_scale, y, rows, cols);
    return check_launch("gemv_int8_simt");
}

}  // namespace tllm
