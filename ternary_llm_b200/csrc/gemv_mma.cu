// Streaming ternary GEMV on the packed layout (packed_layout.cuh), sm_100a.
//
// The GEMV is HBM-bound: 2.125 bits per weight must stream at several TB/s, which
// leaves about 1.5 issue slots per weight per lane.  A masked add per weight on
// the CUDA cores costs 3-5, so the +x/-x/0 selection runs on the tensor cores
// instead: one PRMT expands four packed weights into an INT8 {-1,0,+1} operand
// register of mma.sync.m16n8k32 (A = 16 weight rows x 32 columns), and the B
// operand carries the activations.  Integer MMA keeps every group sum exact.
//
//   FP16 activations: each scale group of 128 activations is converted once per
//   CTA to block fixed point, q = rint(x * 2^(22-e)) with 2^e > max|x| of the
//   group, stored as the three bytes of q + 2^23 (unsigned digits d0,d1,d2).  The
//   B columns of one batch element are [d0 d1 | d2 1]; the column of ones yields
//   sum(t), which removes the 2^23 offset:  sum t*q = D0 + 256*D1 + 65536*(D2 -
//   128*S).  The group sum is exact in INT32 (|sum| <= 2^30); it is converted to
//   FP32 once and multiplied by scale * 2^(e-22).  Rounding x to 23 bits below the
//   group maximum is at the level of FP32 accumulation rounding itself.
//   INT8 activations (ternary_gemv_int8 semantics): B is the int8 vector as is.
//
// Work decomposition: a unit is one 16-row block x 4 scale groups (2176 bytes of
// packed weights).  Units are dealt to CTAs in contiguous, equal ranges (one CTA
// per SM), so K is split across CTAs where rows alone would not balance 148 SMs;
// inside a CTA the units go round-robin to 16 warps.  Each warp streams its units
// through a private cp.async ring (no cross-warp synchronisation on the data
// path).  Per-unit partial sums are reduced in a fixed order; a 16-row block that
// spans two or more CTAs is finished by whichever CTA arrives last, which sums
// the partial records in CTA order, so results do not depend on timing.
//
// Launches carry the programmatic-dependent-launch attribute: the weight prefetch
// is issued before griddepcontrol.wait (weights are constants), activations are
// read and outputs written after it.  CTAs are sized (512 threads, <= 64
// registers, about half of shared memory) so that the next GEMV's CTAs can become
// resident while this one drains.
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "packed_layout.cuh"

namespace tllm {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kUnitGroups = 4;                       // scale groups per unit
constexpr int kUnitBytes = kUnitGroups * kTileBytes; // 2176
constexpr int kRing = 2;                             // units in flight per warp
constexpr int kTickets = 64;                         // independent scratch regions
constexpr int kMaxCtas = 256;

enum Mode { kF16B1 = 0, kF16B2 = 1, kI8 = 2 };

struct GemvArgs {
    const uint8_t* packed;
    const void* x;          // half [batch, cols] or int8 [cols]
    half* y;                // half [batch, rows]
    float in_scale;         // INT8 mode: activation scale
    int rows, cols, groups; // groups = cols / 128
    int upr;                // units per row block = ceil(groups / 4)
    int nrb;                // row blocks = ceil(rows / 16)
    int batch;              // 1 or 2 vectors handled by this launch
    long long total_units;
    int max_units_per_cta;
    float* ws;              // [gridDim.x][2][16][2] partial records of this ticket
    int* counters;          // [nrb] arrival counters of this ticket (zero between launches)
    // shared memory carve-up (byte offsets)
    int off_xfac, off_part, off_ring, off_flags;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t prmt(uint32_t lo, uint32_t hi, uint32_t sel)
{
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(lo), "r"(hi), "r"(sel));
    return r;
}

template <bool BSIGNED>
__device__ __forceinline__ void imma(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                     uint32_t b0, uint32_t b1)
{
    if (BSIGNED)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// First unit index of CTA c when `total` units are dealt to `n` CTAs.
__host__ __device__ inline long long cta_start(long long c, long long total, long long n) { return c * total / n; }
// CTA that owns unit u.
__host__ __device__ inline int cta_of_unit(long long u, long long total, long long n)
{
    return (int)(((u + 1) * n - 1) / total);
}

// ---------------------------------------------------------------------------
// Activation staging
// ---------------------------------------------------------------------------
// FP16 -> block fixed point digits in B-fragment order.  LANES = 16 (one vector,
// columns [d0 d1 d2 1]) or 32 (two vectors).  xdig is uint32 [groups][4 steps][LANES][2].
template <int LANES>
__device__ __forceinline__ void stage_x_f16(const half* __restrict__ x, int cols, int groups, int batch,
                                            uint32_t* xdig, float* xfac, int warp, int lane)
{
    for (int g = warp; g < groups; g += kWarps) {
        for (int b = 0; b < batch; b++) {
            const uint2 raw = *reinterpret_cast<const uint2*>(x + (size_t)b * cols + (size_t)g * kGroup + lane * 4);
            const float2 v01 = __half22float2(*reinterpret_cast<const half2*>(&raw.x));
            const float2 v23 = __half22float2(*reinterpret_cast<const half2*>(&raw.y));
            float m = fmaxf(fmaxf(fabsf(v01.x), fabsf(v01.y)), fmaxf(fabsf(v23.x), fabsf(v23.y)));
            m = warp_max(m);
            // 2^e > m; FP16 inputs keep e within [-23, 16]
            int e = (int)((__float_as_uint(m) >> 23) & 0xffu) - 126;
            e = max(e, -24);
            const float up = (m > 0.f) ? __uint_as_float((uint32_t)(22 - e + 127) << 23) : 0.f;
            const float dn = (m > 0.f) ? __uint_as_float((uint32_t)(e - 22 + 127) << 23) : 0.f;
            const uint32_t q0 = (uint32_t)(__float2int_rn(v01.x * up) + (1 << 23));
            const uint32_t q1 = (uint32_t)(__float2int_rn(v01.y * up) + (1 << 23));
            const uint32_t q2 = (uint32_t)(__float2int_rn(v23.x * up) + (1 << 23));
            const uint32_t q3 = (uint32_t)(__float2int_rn(v23.y * up) + (1 << 23));
            const uint32_t u = __byte_perm(q0, q1, 0x5140), v = __byte_perm(q2, q3, 0x5140);
            const uint32_t r = __byte_perm(q0, q1, 0x0062), s = __byte_perm(q2, q3, 0x0062);
            const uint32_t w0 = __byte_perm(u, v, 0x5410), w1 = __byte_perm(u, v, 0x7632);
            const uint32_t w2 = __byte_perm(r, s, 0x5410);
            // lane holds group columns 4*lane .. 4*lane+3: step m = lane/8, k-slot 4*(lane%8)
            const int m4 = lane >> 3, tq = lane & 7;
            uint32_t* base = xdig + (((size_t)g * 4 + m4) * LANES) * 2 + (tq & 3) * 2 + (tq >> 2);
            const int c0 = b * 4;                       // columns 4b .. 4b+3 of this vector
            base[(c0 + 0) * 8] = w0;
            base[(c0 + 1) * 8] = w1;
            base[(c0 + 2) * 8] = w2;
            base[(c0 + 3) * 8] = 0x01010101u;
            if (lane == 0) xfac[b * groups + g] = dn;
        }
    }
}

// ---------------------------------------------------------------------------
// Kernel
// ---------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(kThreads, 2) gemv_packed_kernel(const GemvArgs a)
{
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr bool I8 = (MODE == kI8);
    constexpr int LANES = (MODE == kF16B2) ? 32 : 16;

    asm volatile("griddepcontrol.launch_dependents;");

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nctas = gridDim.x;
    const long long u0 = cta_start(blockIdx.x, a.total_units, nctas);
    const long long u1 = cta_start(blockIdx.x + 1, a.total_units, nctas);
    const int nunits = (int)(u1 - u0);

    uint32_t* xstage = reinterpret_cast<uint32_t*>(smem);              // digits, or the int8 vector
    float* xfac = reinterpret_cast<float*>(smem + a.off_xfac);
    float* part = reinterpret_cast<float*>(smem + a.off_part);         // [unit][16 rows][2]
    uint8_t* ring = smem + a.off_ring + (size_t)warp * kRing * kUnitBytes;
    int* flags = reinterpret_cast<int*>(smem + a.off_flags);

    // ---- weight prefetch: this warp's first kRing units -----------------------
    auto unit_src = [&](int i, int& ng) -> const uint8_t* {
        const long long u = u0 + i;
        const int rb = (int)(u / a.upr), c = (int)(u % a.upr);
        const int g0 = c * kUnitGroups;
        ng = min(kUnitGroups, a.groups - g0);
        return a.packed + ((size_t)rb * a.groups + g0) * kTileBytes;
    };
    auto issue = [&](int i, int slot) {
        if (i < nunits) {
            int ng;
            const uint8_t* src = unit_src(i, ng);
            const uint32_t dst = smem_addr(ring + (size_t)slot * kUnitBytes);
            const int chunks = ng * (kTileBytes / 16);
            for (int c = lane; c < chunks; c += 32) cp_async16(dst + c * 16, src + (size_t)c * 16);
        }
        cp_async_commit();     // one group per slot fill, possibly empty
    };
#pragma unroll
    for (int s = 0; s < kRing; s++) issue(warp + s * kWarps, s);

    // ---- everything below may depend on the previous kernel in the stream -------
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (I8) {
        const int n16 = a.cols / 16;
        const uint4* src = reinterpret_cast<const uint4*>(a.x);
        for (int i = tid; i < n16; i += kThreads) reinterpret_cast<uint4*>(xstage)[i] = __ldg(src + i);
    } else {
        stage_x_f16<LANES>(reinterpret_cast<const half*>(a.x), a.cols, a.groups, a.batch, xstage, xfac, warp, lane);
    }
    __syncthreads();

    // ---- per-lane constants ------------------------------------------------------
    const int t = lane & 3, gq = lane >> 2;
    int mulA, mulB;          // p = D[odd column] * mulA + D[even column] * mulB
    if (I8) {
        mulA = 0;
        mulB = (t == 0) ? 1 : 0;
    } else {
        const bool live = (MODE == kF16B2) ? ((t >> 1) < a.batch) : (t < 2);
        mulA = !live ? 0 : ((t & 1) ? -(1 << 23) : 256);
        mulB = !live ? 0 : ((t & 1) ? 65536 : 1);
    }
    const int bsel = (MODE == kF16B2) ? (t >> 1) : 0;
    const float* xf = xfac + bsel * a.groups;
    const int xlane = (LANES == 32) ? lane : (lane & 15);

    // ---- main loop: this warp's units -----------------------------------------
    int it = 0;
    for (int i = warp; i < nunits; i += kWarps, it++) {
        const int slot = it % kRing;
        cp_async_wait<kRing - 1>();
        __syncwarp();
        int ng;
        const long long u = u0 + i;
        const int g0 = (int)(u % a.upr) * kUnitGroups;
        ng = min(kUnitGroups, a.groups - g0);
        const uint8_t* tile = ring + (size_t)slot * kUnitBytes;
        float acc0 = 0.f, acc1 = 0.f;       // rows gq and gq+8

#pragma unroll 2
        for (int j = 0; j < ng; j++) {
            const uint8_t* tp = tile + j * kTileBytes;
            const uint2 ca = *reinterpret_cast<const uint2*>(tp + lane * 8);
            const uint2 cb = *reinterpret_cast<const uint2*>(tp + 256 + lane * 8);
            const half2 sc2 = *reinterpret_cast<const half2*>(tp + kTileCodeBytes + gq * 4);
            const int g = g0 + j;
            int dE[4] = {0, 0, 0, 0}, dO[4] = {0, 0, 0, 0};
#pragma unroll
            for (int m = 0; m < 4; m++) {
                const uint32_t wa = (m < 2) ? ca.x : ca.y, wb = (m < 2) ? cb.x : cb.y;
                const uint32_t s0 = (m & 1) ? (wa >> 16) : wa, s1 = (m & 1) ? (wb >> 16) : wb;
                const uint32_t a0 = prmt(kTabA_lo, kTabA_hi, s0), a2 = prmt(kTabB_lo, kTabB_hi, s0);
                const uint32_t a1 = prmt(kTabA_lo, kTabA_hi, s1), a3 = prmt(kTabB_lo, kTabB_hi, s1);
                uint32_t b0, b1;
                if (I8) {
                    const uint32_t* xw = xstage + g * 32 + m * 8 + t;
                    b0 = xw[0];
                    b1 = xw[4];
                } else {
                    const uint2 bb = *reinterpret_cast<const uint2*>(xstage + (((size_t)g * 4 + m) * LANES + xlane) * 2);
                    b0 = bb.x;
                    b1 = bb.y;
                }
                if (m & 1) imma<I8>(dO, a0, a1, a2, a3, b0, b1);
                else imma<I8>(dE, a0, a1, a2, a3, b0, b1);
            }
            const int p0 = (dE[1] + dO[1]) * mulA + (dE[0] + dO[0]) * mulB;
            const int p1 = (dE[3] + dO[3]) * mulA + (dE[2] + dO[2]) * mulB;
            const float2 sc = __half22float2(sc2);
            const float f = I8 ? 1.0f : xf[g];
            acc0 = fmaf((float)p0, sc.x * f, acc0);
            acc1 = fmaf((float)p1, sc.y * f, acc1);
        }
        // lanes t and t^1 hold the two digit halves of one vector
        acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
        acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
        if (I8 || MODE == kF16B1) {
            if (t == 0) {
                part[((size_t)i * 16 + gq) * 2] = acc0;
                part[((size_t)i * 16 + gq + 8) * 2] = acc1;
            }
        } else if ((t & 1) == 0) {
            part[((size_t)i * 16 + gq) * 2 + (t >> 1)] = acc0;
            part[((size_t)i * 16 + gq + 8) * 2 + (t >> 1)] = acc1;
        }
        __syncwarp();
        issue(i + kRing * kWarps, slot);
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- reduction over units, row block by row block ------------------------------
    if (nunits == 0) return;
    const int nb = (MODE == kF16B2) ? a.batch : 1;
    const int rb_first = (int)(u0 / a.upr), rb_last = (int)((u1 - 1) / a.upr);
    const float oscale = I8 ? a.in_scale : 1.0f;
    float* myrec = a.ws + (size_t)blockIdx.x * 2 * 32;
    if (tid < 2) flags[tid] = 0;
    __syncthreads();

    for (int rb = rb_first + (tid >> 5); rb <= rb_last; rb += kWarps) {
        const int row = lane >> 1, b = lane & 1;
        const long long ua = max(u0, (long long)rb * a.upr), ub = min(u1, (long long)(rb + 1) * a.upr);
        float s = 0.f;
        for (long long u = ua; u < ub; u++) s += part[((size_t)(u - u0) * 16 + row) * 2 + b];
        const bool full = (ua == (long long)rb * a.upr) && (ub == (long long)(rb + 1) * a.upr);
        if (full) {
            const int r = rb * 16 + row;
            if (r < a.rows && b < nb) a.y[(size_t)b * a.rows + r] = __float2half_rn(s * oscale);
        } else {
            const int k = (rb == rb_first) ? 0 : 1;
            myrec[k * 32 + lane] = s;
            __threadfence();
            __syncwarp();
            if (lane == 0) {
                const int c_a = cta_of_unit((long long)rb * a.upr, a.total_units, nctas);
                const int c_b = cta_of_unit((long long)(rb + 1) * a.upr - 1, a.total_units, nctas);
                const int prev = atomicAdd(a.counters + rb, 1);
                flags[k] = (prev == c_b - c_a) ? 1 : 0;
            }
            __syncwarp();
            if (flags[k]) {                       // last contributor: finish the row block
                __threadfence();
                const int c_a = cta_of_unit((long long)rb * a.upr, a.total_units, nctas);
                const int c_b = cta_of_unit((long long)(rb + 1) * a.upr - 1, a.total_units, nctas);
                float tot = 0.f;
                for (int c = c_a; c <= c_b; c++) {
                    const int c_first_rb = (int)(cta_start(c, a.total_units, nctas) / a.upr);
                    const int kk = (rb == c_first_rb) ? 0 : 1;
                    tot += __ldcg(a.ws + ((size_t)c * 2 + kk) * 32 + lane);
                }
                const int r = rb * 16 + row;
                if (r < a.rows && b < nb) a.y[(size_t)b * a.rows + r] = __float2half_rn(tot * oscale);
                if (lane == 0) a.counters[rb] = 0;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Repack: reference layout -> packed layout, and back
// ---------------------------------------------------------------------------
__device__ __forceinline__ int tern_at(const uint32_t* nz, const uint32_t* sg, int rows, int wpr, int r, int k)
{
    if (r >= rows) return 0;
    const uint32_t a = nz[(size_t)r * wpr + (k >> 5)], s = sg[(size_t)r * wpr + (k >> 5)];
    const int bit = k & 31;
    return (int)((a >> bit) & 1u) * (2 * (int)((s >> bit) & 1u) - 1);
}

// one thread per (tile, row, lane t): writes its two code words; thread t == 0 also
// writes the row's scale.  Counts sign bits that have no nonzero bit.
__global__ void repack_kernel(const uint32_t* __restrict__ nz, const uint32_t* __restrict__ sg,
                              const half* __restrict__ scales, uint8_t* __restrict__ packed,
                              int rows, int cols, int* __restrict__ noncanon)
{
    const int groups = cols / kGroup, wpr = cols / 32;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long ntiles = (long long)((rows + 15) / 16) * groups;
    if (idx >= ntiles * 64) return;
    const long long tile = idx / 64;
    const int r16 = (int)(idx % 64) / 4, t = (int)(idx % 4);
    const int rb = (int)(tile / groups), g = (int)(tile % groups);
    const int r = rb * 16 + r16;
    uint32_t w[2] = {0, 0};
    for (int m = 0; m < 4; m++) {
        uint32_t sel = 0;
        for (int n = 0; n < 4; n++) {
            const int ka = g * kGroup + 32 * m + 4 * t + n, kb = ka + 16;
            sel |= pair_code(tern_at(nz, sg, rows, wpr, r, ka), tern_at(nz, sg, rows, wpr, r, kb)) << (4 * n);
        }
        w[m >> 1] |= sel << (16 * (m & 1));
    }
    uint8_t* tp = packed + (size_t)tile * kTileBytes;
    *reinterpret_cast<uint2*>(tp + (r16 * 4 + t) * 8) = make_uint2(w[0], w[1]);
    if (r < rows) {
        const uint32_t stray = sg[(size_t)r * wpr + g * 4 + t] & ~nz[(size_t)r * wpr + g * 4 + t];
        if (stray) atomicAdd(noncanon, __popc(stray));
    }
    if (t == 0) {
        const half s = (r < rows) ? scales[(size_t)r * groups + g] : __float2half(0.f);
        const int pos = (r16 < 8) ? 2 * r16 : 2 * (r16 - 8) + 1;
        reinterpret_cast<half*>(tp + kTileCodeBytes)[pos] = s;
    }
}

// one thread per (row, mask word): rebuilds canonical nonzero/sign words; the
// thread of word 0 of each group also restores the scale.
__global__ void unpack_kernel(const uint8_t* __restrict__ packed, uint32_t* __restrict__ nz,
                              uint32_t* __restrict__ sg, half* __restrict__ scales, int rows, int cols)
{
    const int groups = cols / kGroup, wpr = cols / 32;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)rows * wpr) return;
    const int r = (int)(idx / wpr), wd = (int)(idx % wpr);
    const int g = wd / 4, m = wd % 4;          // word wd covers group columns 32m .. 32m+31 = MMA step m
    const uint8_t* tp = packed + ((size_t)(r / 16) * groups + g) * kTileBytes;
    const int r16 = r % 16;
    uint32_t a = 0, s = 0;
    for (int t = 0; t < 4; t++) {
        const uint2 cw = *reinterpret_cast<const uint2*>(tp + (r16 * 4 + t) * 8);
        const uint32_t word = (m < 2) ? cw.x : cw.y;
        const uint32_t sel = (m & 1) ? (word >> 16) : (word & 0xffffu);
        for (int n = 0; n < 4; n++) {
            int ta, tb;
            pair_decode((sel >> (4 * n)) & 0xfu, ta, tb);
            const int ba = 4 * t + n, bb = 16 + 4 * t + n;
            if (ta) a |= 1u << ba;
            if (ta > 0) s |= 1u << ba;
            if (tb) a |= 1u << bb;
            if (tb > 0) s |= 1u << bb;
        }
    }
    nz[idx] = a;
    sg[idx] = s;
    if (m == 0) {
        const int pos = (r16 < 8) ? 2 * r16 : 2 * (r16 - 8) + 1;
        scales[(size_t)r * groups + g] = reinterpret_cast<const half*>(tp + kTileCodeBytes)[pos];
    }
}

// ---------------------------------------------------------------------------
// Host side: scratch, registry, launch
// ---------------------------------------------------------------------------
struct DeviceScratch {
    float* ws = nullptr;       // [kTickets][kMaxCtas][2][32]
    int* counters = nullptr;   // [kTickets][kMaxRowBlocks]
    int* misc = nullptr;       // [0] non-canonical bit counter of the last prepare
    int sms = 0;
    unsigned ticket = 0;
    bool attr_set = false;
};
constexpr int kMaxRowBlocks = 1 << 16;          // rows up to 1,048,576
static DeviceScratch g_scratch[64];
static std::mutex g_mu;

static int get_scratch(DeviceScratch** out)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(TLLM_ERR_DEVICE, "no usable current device");
    DeviceScratch& s = g_scratch[dev];
    if (!s.ws) {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!s.ws) {
            // First use on this device: allocate and zero the scratch.  Must not happen
            // inside a stream capture; make one call per device before capturing.
            cudaDeviceGetAttribute(&s.sms, cudaDevAttrMultiProcessorCount, dev);
            float* ws = nullptr;
            if (cudaMalloc(&ws, (size_t)kTickets * kMaxCtas * 64 * sizeof(float)) != cudaSuccess ||
                cudaMalloc(&s.counters, (size_t)kTickets * kMaxRowBlocks * sizeof(int)) != cudaSuccess ||
                cudaMalloc(&s.misc, 64) != cudaSuccess)
                return fail(TLLM_ERR_LAUNCH, "scratch allocation failed: %s", cudaGetErrorString(cudaGetLastError()));
            cudaMemset(s.counters, 0, (size_t)kTickets * kMaxRowBlocks * sizeof(int));
            cudaMemset(s.misc, 0, 64);
            cudaDeviceSynchronize();
            s.ws = ws;
        }
    }
    *out = &s;
    return TLLM_OK;
}

struct Registered { const uint8_t* packed; int rows, cols; };
static std::unordered_map<const void*, Registered> g_registry;
static std::mutex g_reg_mu;

const uint8_t* lookup_packed(const void* nz, int rows, int cols)
{
    std::lock_guard<std::mutex> lk(g_reg_mu);
    auto it = g_registry.find(nz);
    if (it == g_registry.end() || it->second.rows != rows || it->second.cols != cols) return nullptr;
    return it->second.packed;
}

size_t packed_bytes(int rows, int cols)
{
    return (size_t)((rows + 15) / 16) * (size_t)(cols / kGroup) * kTileBytes;
}

template <int MODE>
static int launch_mode(const GemvArgs& a, int grid, size_t smem, cudaStream_t stream, DeviceScratch* s)
{
    static bool attr[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr[dev]) {
        cudaFuncSetAttribute(gemv_packed_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        attr[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_packed_kernel<MODE>, a);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(TLLM_ERR_LAUNCH, "gemv_packed launch: %s", cudaGetErrorString(e));
    }
    (void)s;
    return TLLM_OK;
}

// x: half [batch, cols] (mode f16) or int8 [cols]; batch 1..2 per launch.
static int launch_packed_once(const uint8_t* packed, const void* x, half* y, float in_scale, int mode,
                              int batch, int rows, int cols, cudaStream_t stream)
{
    DeviceScratch* s = nullptr;
    int st = get_scratch(&s);
    if (st) return st;
    GemvArgs a = {};
    a.packed = packed;
    a.x = x;
    a.y = y;
    a.in_scale = in_scale;
    a.rows = rows;
    a.cols = cols;
    a.groups = cols / kGroup;
    a.upr = (a.groups + kUnitGroups - 1) / kUnitGroups;
    a.nrb = (rows + 15) / 16;
    a.batch = batch;
    a.total_units = (long long)a.nrb * a.upr;
    if (a.nrb > kMaxRowBlocks) return fail(TLLM_ERR_SHAPE, "rows=%d exceeds %d", rows, kMaxRowBlocks * 16);
    int grid = s->sms < kMaxCtas ? s->sms : kMaxCtas;
    if (a.total_units < grid) grid = (int)a.total_units;
    a.max_units_per_cta = (int)((a.total_units + grid - 1) / grid) + 1;
    unsigned ticket;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        ticket = s->ticket++ % kTickets;
    }
    a.ws = s->ws + (size_t)ticket * kMaxCtas * 64;
    a.counters = s->counters + (size_t)ticket * kMaxRowBlocks;
    // shared memory: activations | xfac | partials | ring | flags
    size_t xbytes;
    if (mode == kI8) xbytes = (size_t)cols;
    else xbytes = (size_t)a.groups * 4 * ((mode == kF16B2) ? 32 : 16) * 8;
    size_t off = (xbytes + 15) & ~(size_t)15;
    a.off_xfac = (int)off;
    off += (size_t)2 * a.groups * sizeof(float);
    off = (off + 15) & ~(size_t)15;
    a.off_part = (int)off;
    off += (size_t)a.max_units_per_cta * 32 * sizeof(float);
    off = (off + 15) & ~(size_t)15;
    a.off_ring = (int)off;
    off += (size_t)kWarps * kRing * kUnitBytes;
    a.off_flags = (int)off;
    off += 16;
    if (off > 227 * 1024)
        return fail(TLLM_ERR_SHAPE, "cols=%d needs %zu bytes of shared memory (limit 232448)", cols, off);
    switch (mode) {
        case kF16B1: return launch_mode<kF16B1>(a, grid, off, stream, s);
        case kF16B2: return launch_mode<kF16B2>(a, grid, off, stream, s);
        default: return launch_mode<kI8>(a, grid, off, stream, s);
    }
}

int launch_gemv_packed(const uint8_t* packed, const half* x, half* y, int batch, int rows, int cols,
                       cudaStream_t stream)
{
    // two vectors share one pass over the weights; larger batches take ceil(B/2) passes
    for (int b0 = 0; b0 < batch; b0 += 2) {
        const int nb = (batch - b0 >= 2) ? 2 : 1;
        const int st = launch_packed_once(packed, x + (size_t)b0 * cols, y + (size_t)b0 * rows, 1.0f,
                                          nb == 2 ? kF16B2 : kF16B1, nb, rows, cols, stream);
        if (st) return st;
    }
    return TLLM_OK;
}

int launch_gemv_int8_packed(const uint8_t* packed, const int8_t* xq, float in_scale, half* y, int rows,
                            int cols, cudaStream_t stream)
{
    return launch_packed_once(packed, xq, y, in_scale, kI8, 1, rows, cols, stream);
}

int weight_prepare(const uint32_t* nz, const uint32_t* sg, const half* scales, int rows, int cols,
                   uint8_t* packed, cudaStream_t stream)
{
    DeviceScratch* s = nullptr;
    int st = get_scratch(&s);
    if (st) return st;
    cudaMemsetAsync(s->misc, 0, sizeof(int), stream);
    const long long threads = (long long)((rows + 15) / 16) * (cols / kGroup) * 64;
    repack_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(nz, sg, scales, packed, rows, cols, s->misc);
    if ((st = check_launch("repack"))) return st;
    int stray = 0;
    const cudaError_t e = cudaMemcpyAsync(&stray, s->misc, sizeof(int), cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess || cudaStreamSynchronize(stream) != cudaSuccess)
        return fail(TLLM_ERR_LAUNCH, "prepare: %s", cudaGetErrorString(cudaGetLastError()));
    if (stray)
        return fail(TLLM_ERR_NONCANON, "%d sign bits are set where the nonzero bit is clear; the packed layout "
                    "cannot keep them (they decode to 0 either way)", stray);
    return TLLM_OK;
}

int weight_unpack(const uint8_t* packed, int rows, int cols, uint32_t* nz, uint32_t* sg, half* scales,
                  cudaStream_t stream)
{
    const long long threads = (long long)rows * (cols / 32);
    unpack_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(packed, nz, sg, scales, rows, cols);
    return check_launch("unpack");
}

int weight_register(const void* nz, const uint8_t* packed, int rows, int cols)
{
    std::lock_guard<std::mutex> lk(g_reg_mu);
    g_registry[nz] = Registered{packed, rows, cols};
    return TLLM_OK;
}

int weight_unregister(const void* nz)
{
    std::lock_guard<std::mutex> lk(g_reg_mu);
    g_registry.erase(nz);
    return TLLM_OK;
}

}  // namespace tllm
