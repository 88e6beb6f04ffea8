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
// Work decomposition: the matrix is a linear array of tiles (16 rows x one scale
// group, 544 bytes; row-block major).  Tiles are dealt to CTAs (one per SM) and,
// inside a CTA, to 16 warps in contiguous, equal ranges, so K is split wherever
// rows alone would not balance 148 SMs.  A warp's range is contiguous in memory:
// it arrives through the warp's private two-slot ring of bulk-TMA copies
// (cp.async.bulk + mbarrier, 4 tiles per slot), all issued at kernel start when
// the range fits.  Partial sums of a 16-row block are combined in a fixed order:
// first over the warps of a CTA, then, for a block that spans several CTAs, by
// whichever CTA arrives last, which adds the CTAs' records in CTA order.  Results
// therefore do not depend on timing.
//
// Launches carry the programmatic-dependent-launch attribute: the weight fetch is
// issued before griddepcontrol.wait (weights are constants), activations are read
// and outputs written after it, so a GEMV's weight stream starts while the kernel
// before it in the stream drains.  Every mbarrier wait is bounded; a wait that
// gives up records TLLM_ERR_TIMEOUT in a device flag and the kernel returns.
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "packed_layout.cuh"
#include "launch.cuh"

namespace tllm {

#ifndef TLLM_GEMV_WARPS_LOG2
#define TLLM_GEMV_WARPS_LOG2 4
#endif
constexpr int kWarpsLog2 = TLLM_GEMV_WARPS_LOG2;
constexpr int kWarps = 1 << kWarpsLog2;
constexpr int kThreads = kWarps * 32;
constexpr int kCtasPerSm = (kWarps <= 16) ? 2 : 1;   // co-residency target for __launch_bounds__
constexpr int kSlotTiles = 4;                         // tiles per ring slot
constexpr int kSlotBytes = kSlotTiles * kTileBytes;   // 2176
constexpr int kRing = 2;                              // slots per warp
constexpr int kTickets = 64;                          // independent scratch regions
constexpr int kMaxCtas = 256;
constexpr int kMaxPeers = TLLM_MAX_PEERS;

// kI8Norm / kI8Silu: INT8 arithmetic like kI8, but the activation vector is produced inside
// the kernel's staging phase from FP16 inputs (fused_x.cuh semantics below).
enum Mode { kF16B1 = 0, kF16B2 = 1, kI8 = 2, kI8Norm = 3, kI8Silu = 4, kI8Quant = 5 };

struct GemvArgs {
    const uint8_t* packed;
    const void* x;          // half [batch, cols] or int8 [cols]
    half* y;                // half [batch, rows]
    float in_scale;         // INT8 mode: activation scale
    const float* in_scale_dev;  // INT8 mode: when not null the scale is read from device memory instead
    // kI8Norm: x = quantise(rmsnorm(fx_a (+ fx_b)) * fx_w); the FP16-rounded sum fx_a + fx_b is
    //          written to fx_res_out by CTA 0 when both are given.
    // kI8Silu: x = quantise(silu(fx_a) * fx_b).
    // kI8Quant: x = quantise(fx_a).
    const half* fx_a;
    const half* fx_b;
    const half* fx_w;
    half* fx_res_out;
    float fx_eps;
    int off_xtmp;           // shared memory: half [cols] staging + 64 floats of reduction scratch
    // Several matrices packed back to back and streamed as one (q|k|v, gate|up): row r of the
    // concatenation belongs to segment i with seg_row[i] <= r < seg_row[i + 1] and is written
    // to seg_y[i][r - seg_row[i]].  nseg == 0: one matrix, output y.
    int nseg;
    int seg_row[TLLM_MAX_FUSED + 1];
    half* seg_y[TLLM_MAX_FUSED];
    int rows, cols, groups; // groups = cols / 128 = tiles per row block
    int batch;              // 1 or 2 vectors handled by this launch
    int part_q, part_r;     // items = gridDim.x * part_q + part_r; CTA c owns q (+1 if c < r) items
    int aligned;            // 1: items are whole row blocks (no block spans two CTAs); 0: items are tiles
    int late_release;       // 1: the next kernel in the stream is released after this kernel's own dependency
                            //    wait instead of at its start (see release_rule)
    float* ws;              // [gridDim.x][2][16][2] partial records of this ticket
    int* counters;          // [row blocks] arrival counters of this ticket (zero between launches)
    int* err;               // device error flag (0 = none)
    // shared memory carve-up (byte offsets)
    int off_xfac, off_part, off_ring, off_bar;
    // Fused all-reduce over peer memory (row-parallel shards of a tensor-parallel layer);
    // ar_world == 0 switches it off.  Every rank runs the same launch on its own shard.
    int ar_world, ar_rank, ar_rows_max;
    uint2* ar_recv[kMaxPeers];        // rank d's receive buffer  {value, launch number} [2][world][ar_rows_max]
    unsigned* ar_epoch;               // this rank's launch counters, uint [kMaxCtas]
};

// When a launch releases the next kernel of the stream.  Released at its start, the next
// kernel (and, through it, the one after) becomes resident while this one still runs and
// prefetches its own weights: a long stream of large matrices gains from that depth.  A small
// matrix lives on latencies, and the prefetch traffic of kernels two launches ahead queues in
// front of its activation loads and its final stores; such a launch releases its successor only
// after its own dependency wait, which bounds the look-ahead to one kernel.  Measured on a
// decode step of 2048-wide layers: 2.3 % faster per token with the late release, while the
// 4096-wide benchmark sweep is 4 % slower if its matrices of 16 MB and more are released late.
#ifndef TLLM_LATE_RELEASE_BYTES
#define TLLM_LATE_RELEASE_BYTES (10u << 20)
#endif
static inline int release_rule(int rows, int cols)
{
    const size_t bytes = (size_t)((rows + 15) / 16) * (size_t)(cols / kGroup) * (size_t)kTileBytes;
    return bytes <= (size_t)TLLM_LATE_RELEASE_BYTES ? 1 : 0;
}

#ifdef TLLM_PROFILE_PHASES
__device__ unsigned long long g_phase_ns[kMaxCtas * 16];
__device__ __forceinline__ void phase_mark(int k)
{
    if (threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        g_phase_ns[blockIdx.x * 16 + k] = t;
    }
}
#define PHASE(k) phase_mark(k)
#else
#define PHASE(k)
#endif

// ---- PTX helpers ------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait (about a second at most); false = gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity)
{
#pragma unroll 1
    for (int i = 0; i < (1 << 22); i++)
        if (mbar_try(bar, parity)) return true;
    return false;
}
// Bulk copy global -> this CTA's shared memory, completion counted on `bar`.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t prmt(uint32_t lo, uint32_t hi, uint32_t sel)
{
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(lo), "r"(hi), "r"(sel));
    return r;
}

// D = A.B (+ D when ACC).  The zero accumulator is passed as immediates so that no
// register has to be cleared per group.
template <bool BSIGNED, bool ACC>
__device__ __forceinline__ void imma(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                     uint32_t b0, uint32_t b1)
{
    if (ACC) {
        if (BSIGNED)
            asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
        else
            asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        if (BSIGNED)
            asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
        else
            asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    }
}

// Contiguous equal split of `total` items over `parts`: with q = total / parts and
// r = total % parts (host-computed), part c owns [c*q + min(c,r), ...): the first r
// parts hold q+1 items.  32-bit arithmetic only.
__device__ __forceinline__ int part_start(int c, int q, int r) { return c * q + min(c, r); }
__device__ __forceinline__ int part_of(int u, int q, int r)
{
    const int big = r * (q + 1);
    return (u < big) ? (int)((unsigned)u / (unsigned)(q + 1)) : r + (int)((unsigned)(u - big) / (unsigned)q);
}
// The n tiles of a CTA over its warps: warp w owns [w*n/kWarps, (w+1)*n/kWarps).
__device__ __forceinline__ int warp_start(int w, int n) { return (w * n) >> kWarpsLog2; }
__device__ __forceinline__ int warp_of(int i, int n) { return (int)((unsigned)((i + 1) * kWarps - 1) / (unsigned)n); }

// ---------------------------------------------------------------------------
// Activation staging
// ---------------------------------------------------------------------------
// Three digit words (byte c of four consecutive q values) for one quad of activations.
__device__ __forceinline__ void quad_digits(float v0, float v1, float v2, float v3, float up,
                                            uint32_t& w0, uint32_t& w1, uint32_t& w2)
{
    const uint32_t q0 = (uint32_t)(__float2int_rn(v0 * up) + (1 << 23));
    const uint32_t q1 = (uint32_t)(__float2int_rn(v1 * up) + (1 << 23));
    const uint32_t q2 = (uint32_t)(__float2int_rn(v2 * up) + (1 << 23));
    const uint32_t q3 = (uint32_t)(__float2int_rn(v3 * up) + (1 << 23));
    const uint32_t u = __byte_perm(q0, q1, 0x5140), v = __byte_perm(q2, q3, 0x5140);
    const uint32_t r = __byte_perm(q0, q1, 0x0062), s = __byte_perm(q2, q3, 0x0062);
    w0 = __byte_perm(u, v, 0x5410);
    w1 = __byte_perm(u, v, 0x7632);
    w2 = __byte_perm(r, s, 0x5410);
}

// FP16 -> block fixed point digits in B-operand order.  LANES = 16 (one vector,
// columns [d0 d1 d2 1]) or 32 (two vectors).  xdig is uint32 [groups][2 step pairs]
// [LANES][4]: the four words of lane l = 4*column + t are (b0,b1) of k32 step 2p and
// (b0,b1) of step 2p+1, so one 128-bit shared load feeds two MMAs.
// Each thread converts 8 consecutive activations (one 128-bit load); the 16 lanes of
// a half-warp cover one scale group and agree on its exponent with four shuffles.
template <int LANES>
__device__ __forceinline__ void stage_x_f16(const half* __restrict__ x, int cols, int groups, int batch,
                                            uint32_t* xdig, float* xfac, int tid)
{
    const int per_vec = cols >> 3;                 // 8-element items per vector (multiple of 16)
    const int items = per_vec * batch;
    const int l16 = tid & 15;
    for (int base = 0; base < items; base += kThreads) {
        const int item = base + tid;
        const bool valid = item < items;           // uniform per half-warp
        const int ic = valid ? item : 0;
        const int b = (ic >= per_vec) ? 1 : 0;
        const int e8 = ic - b * per_vec;           // item index inside the vector
        const int g = e8 >> 4;
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + (size_t)b * cols) + e8);
        const float2 f0 = __half22float2(*reinterpret_cast<const half2*>(&raw.x));
        const float2 f1 = __half22float2(*reinterpret_cast<const half2*>(&raw.y));
        const float2 f2 = __half22float2(*reinterpret_cast<const half2*>(&raw.z));
        const float2 f3 = __half22float2(*reinterpret_cast<const half2*>(&raw.w));
        float m = fmaxf(fmaxf(fmaxf(fabsf(f0.x), fabsf(f0.y)), fmaxf(fabsf(f1.x), fabsf(f1.y))),
                        fmaxf(fmaxf(fabsf(f2.x), fabsf(f2.y)), fmaxf(fabsf(f3.x), fabsf(f3.y))));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        // 2^e > m; FP16 inputs keep e within [-23, 16]
        const int e = max((int)((__float_as_uint(m) >> 23) & 0xffu) - 126, -24);
        const float up = (m > 0.f) ? __uint_as_float((uint32_t)(22 - e + 127) << 23) : 0.f;
        const float dn = (m > 0.f) ? __uint_as_float((uint32_t)(e - 22 + 127) << 23) : 0.f;
        uint32_t w[2][3];
        quad_digits(f0.x, f0.y, f1.x, f1.y, up, w[0][0], w[0][1], w[0][2]);
        quad_digits(f2.x, f2.y, f3.x, f3.y, up, w[1][0], w[1][1], w[1][2]);
        if (valid) {
            // quads 2*l16 and 2*l16+1 of the group: k32 step m4 = quad/8, k-slot 4*(quad%8):
            // slots 0..15 are b0 of t = quad%8, slots 16..31 are b1 of t = quad%8 - 4
            const int quad = 2 * l16, m4 = quad >> 3, tq = quad & 7;
            uint32_t* p = xdig + ((g * 2 + (m4 >> 1)) * LANES + b * 16 + (tq & 3)) * 4 + (m4 & 1) * 2 + (tq >> 2);
#pragma unroll
            for (int h = 0; h < 2; h++) {           // second quad: next t, same half
                p[h * 4 + 0 * 16] = w[h][0];
                p[h * 4 + 1 * 16] = w[h][1];
                p[h * 4 + 2 * 16] = w[h][2];
                p[h * 4 + 3 * 16] = 0x01010101u;
            }
            if (l16 == 0) xfac[b * groups + g] = dn;
        }
    }
}

// INT8 activations in shared memory are permuted so that the eight B words a lane needs for
// one scale group (k32 step m, half h: original word 8m + 4h + t of the group's 32) are
// contiguous: slot of original word w = group * 32 + t * 8 + 2m + h.
__device__ __forceinline__ int int8_word_slot(int w)
{
    const int g = w >> 5, r = w & 31;
    return (g << 5) + ((r & 3) << 3) + ((r >> 3) << 1) + ((r >> 2) & 1);
}

// Block-wide reductions over the CTA's kWarps warps; `red` is 33 floats of shared memory.
__device__ __forceinline__ float cta_sum(float v, float* red, int tid)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    if (tid < 32) {
        float t = (tid < kWarps) ? red[tid] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (tid == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ float cta_max(float v, float* red, int tid)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    if (tid < 32) {
        float t = (tid < kWarps) ? red[tid] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
        if (tid == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// The activation vector of an INT8 GEMV produced in place by every CTA from FP16 inputs,
// instead of by a single-CTA kernel in front of the GEMV (a few microseconds of launch
// and dependency latency per operator in a decode step).  Each CTA reads the inputs
// (they sit in L2), so the work is replicated, not the traffic to HBM.
//   kI8Norm  the engine's "residual add, RMSNorm, absmax quantise" (reference
//            src/transformer.cpp:252-268 with kernels/rmsnorm.cu and kernels/activations.cu:88-142):
//            v = half(a + b) (or a when b is null), var = mean(v^2), o = half(v * rsqrt(var + eps) * w),
//            scale = absmax(o) / 127 (1 if zero), q = clamp(rint(o * 127 / absmax)).
//   kI8Silu  "SwiGLU, absmax quantise" (src/transformer.cpp:284-288): o = half(silu(a) * b), then as above.
//   kI8Quant the quantiser alone (src/transformer.cpp:126-136): o = a.
// Returns the activation scale.  tmp: half [cols]; red: 33 floats.
template <int MODE>
__device__ __forceinline__ float stage_x_fused(const GemvArgs& a, int8_t* xq, half* tmp, float* red, int tid)
{
    const int n8 = a.cols >> 3;
    float ss = 0.f, mx = 0.f;
    for (int i = tid; i < n8; i += kThreads) {
        const uint4 ar = *(reinterpret_cast<const uint4*>(a.fx_a) + i);
        uint4 br = make_uint4(0, 0, 0, 0);
        if (MODE != kI8Quant && a.fx_b) br = *(reinterpret_cast<const uint4*>(a.fx_b) + i);
        const half* ah = reinterpret_cast<const half*>(&ar);
        const half* bh = reinterpret_cast<const half*>(&br);
        uint4 st4;
        half* sth = reinterpret_cast<half*>(&st4);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            if (MODE == kI8Silu) {
                // The reference's release build compiles its SiLU with --use_fast_math
                // (CMakeLists.txt:21; kernels/activations.cu:44), i.e. with these intrinsics.  The
                // exact forms cost every CTA about a microsecond per 8192 elements here.
                const float g = __half2float(ah[j]);
                sth[j] = __float2half_rn(__fdividef(g, 1.0f + __expf(-g)) * __half2float(bh[j]));
                mx = fmaxf(mx, fabsf(__half2float(sth[j])));
            } else if (MODE == kI8Quant) {
                sth[j] = ah[j];
                mx = fmaxf(mx, fabsf(__half2float(ah[j])));
            } else {
                sth[j] = a.fx_b ? __float2half_rn(__half2float(ah[j]) + __half2float(bh[j])) : ah[j];
                const float v = __half2float(sth[j]);
                ss += v * v;
            }
        }
        *(reinterpret_cast<uint4*>(tmp) + i) = st4;
        if (MODE == kI8Norm && a.fx_res_out && a.fx_b && blockIdx.x == 0) *(reinterpret_cast<uint4*>(a.fx_res_out) + i) = st4;
    }
    if (MODE == kI8Norm) {
        const float var = cta_sum(ss, red, tid) / (float)a.cols;
        const float rinv = rsqrtf(var + a.fx_eps);
        for (int i = tid; i < n8; i += kThreads) {
            uint4 v4 = *(reinterpret_cast<const uint4*>(tmp) + i);
            const uint4 w4 = __ldg(reinterpret_cast<const uint4*>(a.fx_w) + i);
            half* vh = reinterpret_cast<half*>(&v4);
            const half* wh = reinterpret_cast<const half*>(&w4);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                vh[j] = __float2half_rn(__half2float(vh[j]) * rinv * __half2float(wh[j]));
                mx = fmaxf(mx, fabsf(__half2float(vh[j])));
            }
            *(reinterpret_cast<uint4*>(tmp) + i) = v4;
        }
    }
    const float absmax = cta_max(mx, red, tid);
    const float inv = (absmax > 0.f) ? (127.0f / absmax) : 0.f;
    for (int i = tid; i < n8; i += kThreads) {
        const uint4 v4 = *(reinterpret_cast<const uint4*>(tmp) + i);
        const half* vh = reinterpret_cast<const half*>(&v4);
        uint32_t w[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            uint32_t acc = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int qv = max(-127, min(127, __float2int_rn(__half2float(vh[h * 4 + j]) * inv)));
                acc |= (uint32_t)(qv & 0xff) << (8 * j);
            }
            w[h] = acc;
        }
        reinterpret_cast<uint32_t*>(xq)[int8_word_slot(2 * i)] = w[0];
        reinterpret_cast<uint32_t*>(xq)[int8_word_slot(2 * i + 1)] = w[1];
    }
    return (absmax > 0.f) ? (absmax / 127.0f) : 1.0f;
}

// One tile (one scale group of a 16-row block): four k32 MMA steps.  Returns the
// weighted integer group sums of rows gq (p0) and gq+8 (p1).
//   xq4: FP16 modes, this lane's 128-bit B words of the group (step pairs at [0], [LANES])
//   xw : INT8 mode, this lane's eight B words of the group (int8_word_slot order), 32-byte aligned
template <bool I8, int LANES>
__device__ __forceinline__ void tile_mma(const uint8_t* tp, int lane, const uint4* xq4, const uint32_t* xw,
                                         int mulA, int mulB, int& p0, int& p1)
{
    const uint2 ca = *reinterpret_cast<const uint2*>(tp + lane * 8);
    const uint2 cb = *reinterpret_cast<const uint2*>(tp + 256 + lane * 8);
    uint4 b01, b23;
    if (I8) {
        b01 = *reinterpret_cast<const uint4*>(xw);
        b23 = *reinterpret_cast<const uint4*>(xw + 4);
    } else {
        b01 = xq4[0];
        b23 = xq4[LANES];
    }
    int d[4];
    imma<I8, false>(d, prmt(kTabA_lo, kTabA_hi, ca.x), prmt(kTabA_lo, kTabA_hi, cb.x),
                    prmt(kTabB_lo, kTabB_hi, ca.x), prmt(kTabB_lo, kTabB_hi, cb.x), b01.x, b01.y);
    {
        const uint32_t s0 = ca.x >> 16, s1 = cb.x >> 16;
        imma<I8, true>(d, prmt(kTabA_lo, kTabA_hi, s0), prmt(kTabA_lo, kTabA_hi, s1),
                       prmt(kTabB_lo, kTabB_hi, s0), prmt(kTabB_lo, kTabB_hi, s1), b01.z, b01.w);
    }
    imma<I8, true>(d, prmt(kTabA_lo, kTabA_hi, ca.y), prmt(kTabA_lo, kTabA_hi, cb.y),
                   prmt(kTabB_lo, kTabB_hi, ca.y), prmt(kTabB_lo, kTabB_hi, cb.y), b23.x, b23.y);
    {
        const uint32_t s0 = ca.y >> 16, s1 = cb.y >> 16;
        imma<I8, true>(d, prmt(kTabA_lo, kTabA_hi, s0), prmt(kTabA_lo, kTabA_hi, s1),
                       prmt(kTabB_lo, kTabB_hi, s0), prmt(kTabB_lo, kTabB_hi, s1), b23.z, b23.w);
    }
    if (I8) {
        // every B column carries the same vector, so every accumulator column holds the sum
        p0 = d[0];
        p1 = d[2];
    } else {
        p0 = d[1] * mulA + d[0] * mulB;
        p1 = d[3] * mulA + d[2] * mulB;
    }
}

// Address of output element (vector b, row r) -- see GemvArgs::nseg.
__device__ __forceinline__ half* out_ptr(const GemvArgs& a, int b, int r)
{
    if (a.nseg == 0) return a.y + (size_t)b * a.rows + r;
    int i = 0;
#pragma unroll
    for (int k = 1; k < TLLM_MAX_FUSED; k++)
        if (k < a.nseg && r >= a.seg_row[k]) i = k;
    return a.seg_y[i] + (size_t)b * (a.seg_row[i + 1] - a.seg_row[i]) + (r - a.seg_row[i]);
}

// ---------------------------------------------------------------------------
// Kernel
// ---------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) gemv_packed_kernel(const GemvArgs a)
{
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr bool FUSEDX = (MODE == kI8Norm || MODE == kI8Silu || MODE == kI8Quant);
    constexpr bool I8 = (MODE == kI8 || FUSEDX);
    constexpr int LANES = (MODE == kF16B2) ? 32 : 16;

    if (!a.late_release) asm volatile("griddepcontrol.launch_dependents;");
    PHASE(0);
    TL_MARK(MODE, 0);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = a.groups;
    const int per = a.aligned ? G : 1;                                     // tiles per partition item
    const int t0 = part_start(blockIdx.x, a.part_q, a.part_r) * per;      // first tile of this CTA
    const int n = (a.part_q + ((int)blockIdx.x < a.part_r ? 1 : 0)) * per; // tiles of this CTA
    PHASE(8);
    const int rb_first = (int)((unsigned)t0 / (unsigned)G);
    const int rb_last = (int)((unsigned)(t0 + n - 1) / (unsigned)G);

    uint32_t* xstage = reinterpret_cast<uint32_t*>(smem);              // digits, or the int8 vector
    float* xfac = reinterpret_cast<float*>(smem + a.off_xfac);
    float* part = reinterpret_cast<float*>(smem + a.off_part);         // [segment][16 rows][2]
    const uint32_t ring = smem_addr(smem + a.off_ring) + warp * (kRing * kSlotBytes);
    const uint8_t* ring_p = smem + a.off_ring + warp * (kRing * kSlotBytes);
    const uint32_t bar = smem_addr(smem + a.off_bar) + warp * (kRing * 8);

    // ---- this warp's tile range and its weight fetch ----------------------------
    const int w0 = t0 + warp_start(warp, n), w1 = t0 + warp_start(warp + 1, n);
    const int nw = w1 - w0;                                  // may be 0 for tiny problems
    const int nchunks = (nw + kSlotTiles - 1) / kSlotTiles;
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kRing; s++) mbar_init(bar + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    PHASE(9);
    auto fetch = [&](int chunk) {                            // lane 0 only
        const int first = w0 + chunk * kSlotTiles;
        const uint32_t bytes = (uint32_t)min(kSlotTiles, w1 - first) * kTileBytes;
        const int slot = chunk % kRing;
        mbar_expect_tx(bar + slot * 8, bytes);
        bulk_g2s(ring + slot * kSlotBytes, a.packed + (size_t)first * kTileBytes, bytes, bar + slot * 8);
    };
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kRing; s++)
            if (s < nchunks) fetch(s);
    }

    // ---- everything below may depend on the previous kernel in the stream -------
    PHASE(1);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (a.late_release) asm volatile("griddepcontrol.launch_dependents;");
    PHASE(2);
    TL_MARK(MODE, 1);

    float fused_scale = 1.0f;
    if (FUSEDX) {
        fused_scale = stage_x_fused<MODE>(a, reinterpret_cast<int8_t*>(xstage), reinterpret_cast<half*>(smem + a.off_xtmp),
                                          reinterpret_cast<float*>(smem + a.off_xtmp + (size_t)a.cols * sizeof(half)), tid);
    } else if (I8) {
        const int n16 = a.cols / 16;
        const uint4* src = reinterpret_cast<const uint4*>(a.x);
        for (int i = tid; i < n16; i += kThreads) {
            const uint4 v = __ldg(src + i);
            xstage[int8_word_slot(4 * i)] = v.x;
            xstage[int8_word_slot(4 * i + 1)] = v.y;
            xstage[int8_word_slot(4 * i + 2)] = v.z;
            xstage[int8_word_slot(4 * i + 3)] = v.w;
        }
    } else {
        stage_x_f16<LANES>(reinterpret_cast<const half*>(a.x), a.cols, G, a.batch, xstage, xfac, tid);
    }
    __syncthreads();
    PHASE(3);
    TL_MARK(MODE, 2);

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
    const float* xf = xfac + ((MODE == kF16B2) ? (t >> 1) : 0) * G;
    const uint4* xq4 = reinterpret_cast<const uint4*>(xstage) + ((LANES == 32) ? lane : (lane & 15));
    const uint32_t* xw = xstage + t * 8;

    // ---- main loop: this warp's tiles, four per ring slot --------------------------
    int rb = (int)((unsigned)w0 / (unsigned)G);
    int g = w0 - rb * G;
    int seg = (rb - rb_first) + warp;        // partial-sum slot: unique per (warp, row block), ascending
    float acc0 = 0.f, acc1 = 0.f;            // rows gq and gq+8 of row block rb
    bool dirty = false, ok = true;

    auto flush = [&]() {
        if (!I8) {       // lanes t and t^1 hold the two digit halves of one vector
            acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
            acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
        }
        float* pu = part + seg * 32;
        if (I8 || MODE == kF16B1) {
            if (t == 0) {
                pu[gq * 2] = acc0;
                pu[(gq + 8) * 2] = acc1;
            }
        } else if ((t & 1) == 0) {
            pu[gq * 2 + (t >> 1)] = acc0;
            pu[(gq + 8) * 2 + (t >> 1)] = acc1;
        }
        acc0 = acc1 = 0.f;
        dirty = false;
    };

    for (int c = 0; c < nchunks && ok; c++) {
        const int slot = c % kRing;
        ok = mbar_wait(bar + slot * 8, (uint32_t)(c / kRing) & 1u);
        if (!ok) break;
        const uint8_t* tile = ring_p + slot * kSlotBytes;
        const int nt = min(kSlotTiles, nw - c * kSlotTiles);
        if (nt == kSlotTiles && g + kSlotTiles <= G) {
            // common case: four tiles of one row block, straight-line code with
            // compile-time offsets and four independent MMA chains
            const uint4* xg = xq4 + g * (2 * LANES);
            const uint32_t* xwg = xw + g * 32;
            int p[kSlotTiles][2];
#pragma unroll
            for (int q = 0; q < kSlotTiles; q++)
                tile_mma<I8, LANES>(tile + q * kTileBytes, lane, xg + q * (2 * LANES), xwg + q * 32, mulA, mulB,
                                    p[q][0], p[q][1]);
#pragma unroll
            for (int q = 0; q < kSlotTiles; q++) {
                const float2 sc = __half22float2(
                    *reinterpret_cast<const half2*>(tile + q * kTileBytes + kTileCodeBytes + gq * 4));
                const float f = I8 ? 1.0f : xf[g + q];
                acc0 = fmaf((float)p[q][0], sc.x * f, acc0);
                acc1 = fmaf((float)p[q][1], sc.y * f, acc1);
            }
            g += kSlotTiles;
            dirty = true;
            if (g == G) {
                flush();
                g = 0;
                rb++;
                seg++;
            }
        } else {
            // ragged slot (end of the warp's range or a row-block boundary inside it)
            for (int j = 0; j < nt; j++) {
                const uint8_t* tp = tile + j * kTileBytes;
                int pa0, pa1;
                tile_mma<I8, LANES>(tp, lane, xq4 + g * (2 * LANES), xw + g * 32, mulA, mulB, pa0, pa1);
                const float2 sa = __half22float2(*reinterpret_cast<const half2*>(tp + kTileCodeBytes + gq * 4));
                const float fa = I8 ? 1.0f : xf[g];
                acc0 = fmaf((float)pa0, sa.x * fa, acc0);
                acc1 = fmaf((float)pa1, sa.y * fa, acc1);
                g++;
                dirty = true;
                if (g == G) {                    // row block finished (for this warp)
                    flush();
                    g = 0;
                    rb++;
                    seg++;
                }
            }
        }
        if (c + kRing < nchunks) {           // refill this slot with the chunk two ahead
            __syncwarp();
            if (lane == 0) fetch(c + kRing);
        }
    }
    if (dirty) flush();
    if (!ok && lane == 0) atomicExch(a.err, TLLM_ERR_TIMEOUT);
    PHASE(4);
    TL_MARK(MODE, 3);
    __syncthreads();
    PHASE(5);

    // ---- reduction: warps of this CTA, then CTAs, row block by row block -----------
    const int nb = (MODE == kF16B2) ? a.batch : 1;
    const float oscale = FUSEDX ? fused_scale : (I8 ? (a.in_scale_dev ? __ldg(a.in_scale_dev) : a.in_scale) : 1.0f);
    float* myrec = a.ws + (size_t)blockIdx.x * 64;

    if (a.ar_world > 0) {
        // ---- fused all-reduce: my partial sums go straight into every rank's receive
        // buffer over NVLink as 8-byte {value, launch number} words -- the store of a word
        // is atomic, so the launch number doubles as the arrival flag and no fence or
        // separate flag round is needed.  Each CTA then polls (bounded) its OWN memory for
        // the other ranks' words of the same rows -- every rank runs this launch with the
        // same partition -- and adds the contributions in rank order.  Buffers alternate
        // with the launch parity, so a rank that runs one launch ahead never overwrites
        // words that are still being read.
        const unsigned epoch = a.ar_epoch[blockIdx.x] + 1u;
        const unsigned par = epoch & 1u;
        const size_t slot = (size_t)(par * a.ar_world + a.ar_rank) * a.ar_rows_max;
        for (int r_b = rb_first + warp; r_b <= rb_last; r_b += kWarps) {
            const int ta = max(t0, r_b * G), tb = min(t0 + n, (r_b + 1) * G);
            const int wa = warp_of(ta - t0, n), wb = warp_of(tb - 1 - t0, n);
            float s = 0.f;
            for (int w = wa; w <= wb; w++)
                if (warp_start(w + 1, n) > warp_start(w, n)) s += part[((r_b - rb_first) + w) * 32 + lane];
            const int r = r_b * 16 + (lane >> 1);
            if ((lane & 1) == 0 && r < a.rows) {
                const uint2 word = make_uint2(__float_as_uint(s), epoch);
                for (int d = 0; d < a.ar_world; d++) {
                    uint2* dst = a.ar_recv[d] + slot + r;
                    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(word.x), "r"(word.y) : "memory");
                }
            }
        }
        const int r_lo = rb_first * 16, r_hi = min(a.rows, (rb_last + 1) * 16);
        const uint2* recv = a.ar_recv[a.ar_rank] + (size_t)par * a.ar_world * a.ar_rows_max;
        bool ok_ar = true;
        for (int r = r_lo + tid; r < r_hi; r += kThreads) {
            float v = 0.f;
            for (int d = 0; d < a.ar_world; d++) {
                const uint2* src = recv + (size_t)d * a.ar_rows_max + r;
                uint32_t val = 0, tag = 0;
#pragma unroll 1
                for (int i = 0; i < (1 << 21); i++) {       // about half a second at most
                    asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(val), "=r"(tag) : "l"(src) : "memory");
                    if (tag == epoch) break;
                    __nanosleep(32);
                }
                ok_ar = ok_ar && (tag == epoch);
                v += __uint_as_float(val);
            }
            a.y[r] = __float2half_rn(v);
        }
        if (!ok_ar) atomicExch(a.err, TLLM_ERR_TIMEOUT);
        __syncthreads();
        if (tid == 0) a.ar_epoch[blockIdx.x] = epoch;
        PHASE(6);
        return;
    }

    for (int r_b = rb_first + warp; r_b <= rb_last; r_b += kWarps) {
        const int row = lane >> 1, b = lane & 1;
        const int ta = max(t0, r_b * G), tb = min(t0 + n, (r_b + 1) * G);     // this CTA's tiles of the block
        const int wa = warp_of(ta - t0, n), wb = warp_of(tb - 1 - t0, n);
        float s = 0.f;
        for (int w = wa; w <= wb; w++)
            if (warp_start(w + 1, n) > warp_start(w, n))       // warps without tiles wrote nothing
                s += part[((r_b - rb_first) + w) * 32 + lane];
        const bool full = (tb - ta == G);
        const int r = r_b * 16 + row;
        if (full) {
            if (r < a.rows && b < nb) *out_ptr(a, b, r) = __float2half_rn(s * oscale);
        } else {
            // this row block is shared with neighbouring CTAs: publish the partial sums;
            // the contributor that arrives last adds all records in CTA order
            const int k = (r_b == rb_first) ? 0 : 1;
            myrec[k * 32 + lane] = s;
            __threadfence();
            __syncwarp();
            int c_a = 0, c_b = 0, last = 0;
            if (lane == 0) {
                c_a = part_of(r_b * G, a.part_q, a.part_r);
                c_b = part_of((r_b + 1) * G - 1, a.part_q, a.part_r);
                const int prev = atomicAdd(a.counters + r_b, 1);
                last = (prev == c_b - c_a) ? 1 : 0;
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                __threadfence();
                c_a = __shfl_sync(0xffffffffu, c_a, 0);
                c_b = __shfl_sync(0xffffffffu, c_b, 0);
                float tot = 0.f;
                for (int c = c_a; c <= c_b; c++) {
                    // record 0 of a CTA belongs to its first row block, record 1 to its last
                    const int c_rb = (int)((unsigned)part_start(c, a.part_q, a.part_r) / (unsigned)G);
                    tot += __ldcg(a.ws + (size_t)c * 64 + ((r_b == c_rb) ? 0 : 32) + lane);
                }
                if (r < a.rows && b < nb) *out_ptr(a, b, r) = __float2half_rn(tot * oscale);
                if (lane == 0) a.counters[r_b] = 0;
            }
        }
    }
    PHASE(6);
}

// ---------------------------------------------------------------------------
// Column-walk GEMV: one vector, matrices with enough row blocks for all SMs
// ---------------------------------------------------------------------------
// Same arithmetic as gemv_packed_kernel, different traversal.  A CTA owns whole row
// blocks (so no block is shared between CTAs); inside it warp w owns the scale groups
// w, w+16, w+32, ... and walks DOWN the CTA's row blocks for each of them.  The B
// operand of a group (the activations' digits) is loaded into registers once per
// group and reused for every row block, the group's 2^e factor likewise, and each
// warp stages only its own groups' activations in a private piece of shared memory,
// so there is no CTA-wide barrier before the main loop.  Weight tiles arrive through a
// per-warp cp.async ring (RING tiles of 544 bytes).  Up to 8 row blocks are accumulated
// in registers at a time; the 16 warps' partial sums of a row block are added in warp
// order at the end.
constexpr int kMaxFused = TLLM_MAX_FUSED;   // matrices sharing x in one launch (q/k/v, gate/up)

struct CwArgs {
    const uint8_t* packed[kMaxFused];
    half* y[kMaxFused];             // half [rows[i]]
    int rows[kMaxFused];
    int rb_start[kMaxFused + 1];    // first row block of matrix i in the concatenated row-block space
    int count;                      // matrices in this launch
    const void* x;                  // half [cols] or int8 [cols], shared by all matrices
    float in_scale;
    const float* in_scale_dev;      // INT8 mode: scale in device memory when not null
    int cols, groups;
    int part_q, part_r;     // row blocks = gridDim.x * part_q + part_r
    int gpw;                // groups per warp, ceil(groups / kWarps)
    int off_xfac, off_part, off_ring;   // shared memory carve-up; digit staging starts at 0
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Four k32 steps of one tile with all operands in registers.
template <bool I8>
__device__ __forceinline__ void tile_mma_r(uint2 ca, uint2 cb, uint4 b01, uint4 b23, int mulA, int mulB, int& p0, int& p1)
{
    int d[4];
    imma<I8, false>(d, prmt(kTabA_lo, kTabA_hi, ca.x), prmt(kTabA_lo, kTabA_hi, cb.x),
                    prmt(kTabB_lo, kTabB_hi, ca.x), prmt(kTabB_lo, kTabB_hi, cb.x), b01.x, b01.y);
    {
        const uint32_t s0 = ca.x >> 16, s1 = cb.x >> 16;
        imma<I8, true>(d, prmt(kTabA_lo, kTabA_hi, s0), prmt(kTabA_lo, kTabA_hi, s1),
                       prmt(kTabB_lo, kTabB_hi, s0), prmt(kTabB_lo, kTabB_hi, s1), b01.z, b01.w);
    }
    imma<I8, true>(d, prmt(kTabA_lo, kTabA_hi, ca.y), prmt(kTabA_lo, kTabA_hi, cb.y),
                   prmt(kTabB_lo, kTabB_hi, ca.y), prmt(kTabB_lo, kTabB_hi, cb.y), b23.x, b23.y);
    {
        const uint32_t s0 = ca.y >> 16, s1 = cb.y >> 16;
        imma<I8, true>(d, prmt(kTabA_lo, kTabA_hi, s0), prmt(kTabA_lo, kTabA_hi, s1),
                       prmt(kTabB_lo, kTabB_hi, s0), prmt(kTabB_lo, kTabB_hi, s1), b23.z, b23.w);
    }
    p0 = d[1] * mulA + d[0] * mulB;
    p1 = d[3] * mulA + d[2] * mulB;
}

constexpr int kCwBlock = 8;      // row blocks accumulated in registers at a time

template <int MODE, int RING>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) gemv_cw_kernel(const CwArgs a)
{
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr bool I8 = (MODE == kI8);
    static_assert(MODE != kF16B2, "one vector only");
    static_assert((RING & (RING - 1)) == 0 && RING >= 2, "ring depth must be a power of two");

    asm volatile("griddepcontrol.launch_dependents;");
    PHASE(0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = a.groups;
    const int rb0 = part_start(blockIdx.x, a.part_q, a.part_r);
    const int nrb = a.part_q + ((int)blockIdx.x < a.part_r ? 1 : 0);
    const int ngw = (warp < G) ? ((G - warp + kWarps - 1) >> kWarpsLog2) : 0;   // groups of this warp
    // matrix that owns row block R of the concatenated space
    auto which = [&](int R) {
        int i = 0;
#pragma unroll
        for (int j = 1; j < kMaxFused; j++)
            if (j < a.count && R >= a.rb_start[j]) i = j;
        return i;
    };
    const int nblk = (nrb + kCwBlock - 1) / kCwBlock;
    const int ntiles = ngw * nrb;

    uint32_t* stage = reinterpret_cast<uint32_t*>(smem) + warp * a.gpw * 128;   // 512 bytes per group
    float* xfs = reinterpret_cast<float*>(smem + a.off_xfac) + warp * a.gpw;
    float* part = reinterpret_cast<float*>(smem + a.off_part);                  // [row block][warp][32]
    const uint32_t ring = smem_addr(smem + a.off_ring) + warp * (RING * kTileBytes);
    const uint8_t* ring_p = smem + a.off_ring + warp * (RING * kTileBytes);

    // ---- weight fetch, RING-1 tiles ahead of the arithmetic --------------------------
    int fcnt = 0, fblk = 0, fgi = 0, fri = 0;
    auto fetch = [&]() {
        if (fcnt < ntiles) {
            const int rb = rb0 + fblk * kCwBlock + fri, g = warp + (fgi << kWarpsLog2);
            const int mi = which(rb);
            const uint8_t* src = a.packed[mi] + ((size_t)(rb - a.rb_start[mi]) * G + g) * kTileBytes;
            const uint32_t dst = ring + (fcnt & (RING - 1)) * kTileBytes;
            cp_async16(dst + lane * 16, src + lane * 16);
            if (lane < kTileBytes / 16 - 32) cp_async16(dst + 512 + lane * 16, src + 512 + lane * 16);
            fcnt++;
            if (++fri == min(kCwBlock, nrb - fblk * kCwBlock)) {
                fri = 0;
                if (++fgi == ngw) {
                    fgi = 0;
                    fblk++;
                }
            }
        }
        cp_async_commit();       // one group per tile slot, possibly empty
    };
#pragma unroll
    for (int s = 0; s < RING - 1; s++) fetch();

    // ---- everything below may depend on the previous kernel in the stream -------
    PHASE(1);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    PHASE(2);

    if (!I8) {
        // this warp's groups only: digits in B-operand order, 512 bytes per group
        const half* x = reinterpret_cast<const half*>(a.x);
        for (int gi = 0; gi < ngw; gi++) {
            const int g = warp + (gi << kWarpsLog2);
            const uint2 raw = __ldg(reinterpret_cast<const uint2*>(x + (size_t)g * kGroup) + lane);
            const float2 f0 = __half22float2(*reinterpret_cast<const half2*>(&raw.x));
            const float2 f1 = __half22float2(*reinterpret_cast<const half2*>(&raw.y));
            float m = fmaxf(fmaxf(fabsf(f0.x), fabsf(f0.y)), fmaxf(fabsf(f1.x), fabsf(f1.y)));
            m = warp_max(m);
            const int e = max((int)((__float_as_uint(m) >> 23) & 0xffu) - 126, -24);
            const float up = (m > 0.f) ? __uint_as_float((uint32_t)(22 - e + 127) << 23) : 0.f;
            const float dn = (m > 0.f) ? __uint_as_float((uint32_t)(e - 22 + 127) << 23) : 0.f;
            uint32_t w0, w1, w2;
            quad_digits(f0.x, f0.y, f1.x, f1.y, up, w0, w1, w2);
            // quad `lane` of the group: k32 step lane/8, k-slot 4*(lane%8)
            const int m4 = lane >> 3, tq = lane & 7;
            uint32_t* p = stage + ((gi * 2 + (m4 >> 1)) * 16 + (tq & 3)) * 4 + (m4 & 1) * 2 + (tq >> 2);
            p[0 * 16] = w0;
            p[1 * 16] = w1;
            p[2 * 16] = w2;
            p[3 * 16] = 0x01010101u;
            if (lane == 0) xfs[gi] = dn;
        }
    }
    __syncwarp();
    PHASE(3);

    const int t = lane & 3, gq = lane >> 2;
    int mulA, mulB;
    if (I8) {
        mulA = 0;
        mulB = (t == 0) ? 1 : 0;
    } else {
        mulA = (t >= 2) ? 0 : ((t & 1) ? -(1 << 23) : 256);
        mulB = (t >= 2) ? 0 : ((t & 1) ? 65536 : 1);
    }

    int cnt = 0;
    for (int blk = 0; blk < nblk; blk++) {
        const int nr = min(kCwBlock, nrb - blk * kCwBlock);
        float acc[kCwBlock][2];
#pragma unroll
        for (int r = 0; r < kCwBlock; r++) acc[r][0] = acc[r][1] = 0.f;

        for (int gi = 0; gi < ngw; gi++) {
            uint4 b01, b23;
            float f;
            if (I8) {
                const uint32_t* xw = reinterpret_cast<const uint32_t*>(a.x) + (warp + (gi << kWarpsLog2)) * 32 + t;
                b01 = make_uint4(__ldg(xw), __ldg(xw + 4), __ldg(xw + 8), __ldg(xw + 12));
                b23 = make_uint4(__ldg(xw + 16), __ldg(xw + 20), __ldg(xw + 24), __ldg(xw + 28));
                f = 1.0f;
            } else {
                const uint4* s4 = reinterpret_cast<const uint4*>(stage) + gi * 32 + (lane & 15);
                b01 = s4[0];
                b23 = s4[16];
                f = xfs[gi];
            }
#pragma unroll
            for (int r = 0; r < kCwBlock; r++) {
                if (r < nr) {
                    cp_async_wait<RING - 2>();       // tile `cnt` has landed
                    __syncwarp();                    // ... for all lanes, and tile cnt-1 is no longer read
                    fetch();                         // refill the slot of tile cnt-1
                    const uint8_t* tp = ring_p + (cnt & (RING - 1)) * kTileBytes;
                    const uint2 ca = *reinterpret_cast<const uint2*>(tp + lane * 8);
                    const uint2 cb = *reinterpret_cast<const uint2*>(tp + 256 + lane * 8);
                    const float2 sc = __half22float2(*reinterpret_cast<const half2*>(tp + kTileCodeBytes + gq * 4));
                    int p0, p1;
                    tile_mma_r<I8>(ca, cb, b01, b23, mulA, mulB, p0, p1);
                    acc[r][0] = fmaf((float)p0, sc.x * f, acc[r][0]);
                    acc[r][1] = fmaf((float)p1, sc.y * f, acc[r][1]);
                    cnt++;
                }
            }
        }
        // this warp's sums for the block's row blocks (lanes t and t^1 hold the two digit halves)
#pragma unroll
        for (int r = 0; r < kCwBlock; r++) {
            if (r < nr) {
                const float v0 = acc[r][0] + __shfl_xor_sync(0xffffffffu, acc[r][0], 1);
                const float v1 = acc[r][1] + __shfl_xor_sync(0xffffffffu, acc[r][1], 1);
                if (t == 0 && ngw > 0) {
                    float* pu = part + ((blk * kCwBlock + r) * kWarps + warp) * 32;
                    pu[gq * 2] = v0;
                    pu[(gq + 8) * 2] = v1;
                }
            }
        }
    }
    cp_async_wait<0>();
    PHASE(4);
    __syncthreads();
    PHASE(5);

    // ---- add the warps' partial sums in warp order and store -------------------------
    const float oscale = I8 ? (a.in_scale_dev ? __ldg(a.in_scale_dev) : a.in_scale) : 1.0f;
    const int nwarps_used = min(kWarps, G);
    for (int rbl = warp; rbl < nrb; rbl += kWarps) {
        if ((lane & 1) == 0) {
            float s = 0.f;
            for (int w = 0; w < nwarps_used; w++) s += part[(rbl * kWarps + w) * 32 + lane];
            const int mi = which(rb0 + rbl);
            const int r = (rb0 + rbl - a.rb_start[mi]) * 16 + (lane >> 1);
            if (r < a.rows[mi]) a.y[mi][r] = __float2half_rn(s * oscale);
        }
    }
    PHASE(6);
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
        cudaFuncSetAttribute(gemv_packed_kernel<MODE>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
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
struct SegY {
    int n;
    int rows[TLLM_MAX_FUSED];
    half* y[TLLM_MAX_FUSED];
};

struct FusedX {
    const half* a;
    const half* b;
    const half* w;
    half* res_out;
    float eps;
};

static int launch_packed_once(const uint8_t* packed, const void* x, half* y, float in_scale, int mode,
                              int batch, int rows, int cols, cudaStream_t stream, const float* in_scale_dev = nullptr,
                              const FusedX* fx = nullptr, const SegY* seg = nullptr)
{
    DeviceScratch* s = nullptr;
    int st = get_scratch(&s);
    if (st) return st;
    GemvArgs a = {};
    a.packed = packed;
    a.x = x;
    a.y = y;
    a.in_scale = in_scale;
    a.in_scale_dev = in_scale_dev;
    if (seg) {
        a.nseg = seg->n;
        int r0 = 0;
        for (int i = 0; i < seg->n; i++) {
            a.seg_row[i] = r0;
            a.seg_y[i] = seg->y[i];
            r0 += seg->rows[i];
        }
        for (int i = seg->n; i <= TLLM_MAX_FUSED; i++) a.seg_row[i] = r0;
    }
    if (fx) {
        a.fx_a = fx->a;
        a.fx_b = fx->b;
        a.fx_w = fx->w;
        a.fx_res_out = fx->res_out;
        a.fx_eps = fx->eps;
    }
    a.rows = rows;
    a.cols = cols;
    a.groups = cols / kGroup;
    a.batch = batch;
    const int nrb = (rows + 15) / 16;
    if (nrb > kMaxRowBlocks) return fail(TLLM_ERR_SHAPE, "rows=%d exceeds %d", rows, kMaxRowBlocks * 16);
    if ((long long)nrb * a.groups >= (1ll << 26))
        return fail(TLLM_ERR_SHAPE, "rows=%d cols=%d: more than 2^26 tiles", rows, cols);
    const int tiles = nrb * a.groups;
    int grid = s->sms < kMaxCtas ? s->sms : kMaxCtas;
    // Whole row blocks per CTA when that keeps the SMs at least 80 % evenly loaded: no
    // row block then spans two CTAs and the cross-CTA combine never runs.  Otherwise
    // split at tile granularity (K is split across CTAs).
    const int per_cta_rb = (nrb + grid - 1) / grid;
    a.aligned = (nrb >= grid && (double)nrb / ((double)per_cta_rb * grid) >= 0.8) ? 1 : 0;
    // Fewer row blocks than SMs and short rows (one ring slot per warp at most): such a
    // matrix is a few hundred KB, latency-bound, and the cross-CTA combine would cost more
    // than the idle SMs; one CTA per row block.
    if (nrb < grid && a.groups <= kWarps * kSlotTiles) a.aligned = 1;
    // The same holds with a few more row blocks than SMs when a CTA's share is still at most
    // one ring slot per warp (q|k|v of a small model: 192 row blocks of 16 tiles).
    if (per_cta_rb * a.groups <= kWarps * kSlotTiles) a.aligned = 1;
    const int items = a.aligned ? nrb : tiles;
    if (items < grid) grid = items;
    a.part_q = items / grid;
    a.part_r = items % grid;
    a.late_release = release_rule(rows, cols);
    unsigned ticket;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        ticket = s->ticket++ % kTickets;
    }
    a.ws = s->ws + (size_t)ticket * kMaxCtas * 64;
    a.counters = s->counters + (size_t)ticket * kMaxRowBlocks;
    a.err = s->misc + 1;
    // shared memory: activations | xfac | partial sums | rings | mbarriers
    size_t xbytes;
    const bool fusedx = (mode == kI8Norm || mode == kI8Silu || mode == kI8Quant);
    if (mode == kI8 || fusedx) xbytes = (size_t)cols;
    else xbytes = (size_t)a.groups * 2 * ((mode == kF16B2) ? 32 : 16) * 16;
    size_t off = (xbytes + 15) & ~(size_t)15;
    a.off_xfac = (int)off;
    off += (size_t)2 * a.groups * sizeof(float);
    off = (off + 15) & ~(size_t)15;
    a.off_part = (int)off;
    const int max_rb_per_cta = a.aligned ? (a.part_q + 1) : ((a.part_q + 1 + a.groups - 1) / a.groups + 1);
    off += (size_t)(max_rb_per_cta + kWarps) * 32 * sizeof(float);
    off = (off + 15) & ~(size_t)15;
    a.off_ring = (int)off;
    off += (size_t)kWarps * kRing * kSlotBytes;
    a.off_bar = (int)off;
    off += (size_t)kWarps * kRing * 8;
    if (fusedx) {
        off = (off + 15) & ~(size_t)15;
        a.off_xtmp = (int)off;
        off += (size_t)cols * sizeof(half) + 64 * sizeof(float);
    }
    if (off > 227 * 1024)
        return fail(TLLM_ERR_SHAPE, "rows=%d cols=%d needs %zu bytes of shared memory (limit 232448)", rows, cols, off);
    switch (mode) {
        case kF16B1: return launch_mode<kF16B1>(a, grid, off, stream, s);
        case kF16B2: return launch_mode<kF16B2>(a, grid, off, stream, s);
        case kI8Norm: return launch_mode<kI8Norm>(a, grid, off, stream, s);
        case kI8Silu: return launch_mode<kI8Silu>(a, grid, off, stream, s);
        case kI8Quant: return launch_mode<kI8Quant>(a, grid, off, stream, s);
        default: return launch_mode<kI8>(a, grid, off, stream, s);
    }
}

// Column-walk kernel: usable when whole row blocks balance the SMs and every warp has a group.
static bool cw_eligible_rb(int sms, int nrb, int cols)
{
    const int groups = cols / kGroup;
    int grid = sms < kMaxCtas ? sms : kMaxCtas;
    if (nrb < grid || groups < kWarps) return false;
    const int per = (nrb + grid - 1) / grid;
    return (double)nrb / ((double)per * grid) >= 0.8;
}
static bool cw_eligible(int sms, int rows, int cols) { return cw_eligible_rb(sms, (rows + 15) / 16, cols); }

template <int MODE, int RING>
static int launch_cw_t(const CwArgs& a, int grid, size_t smem, cudaStream_t stream)
{
    static bool attr[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr[dev]) {
        cudaFuncSetAttribute(gemv_cw_kernel<MODE, RING>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        cudaFuncSetAttribute(gemv_cw_kernel<MODE, RING>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
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
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_cw_kernel<MODE, RING>, a);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(TLLM_ERR_LAUNCH, "gemv_cw launch: %s", cudaGetErrorString(e));
    }
    return TLLM_OK;
}

static int launch_cw_multi(int count, const uint8_t* const* packed, half* const* y, const int* rows, const void* x,
                           float in_scale, int mode, int cols, int sms, cudaStream_t stream,
                           const float* in_scale_dev = nullptr)
{
    CwArgs a = {};
    int nrb = 0;
    for (int i = 0; i < count; i++) {
        a.packed[i] = packed[i];
        a.y[i] = y[i];
        a.rows[i] = rows[i];
        a.rb_start[i] = nrb;
        nrb += (rows[i] + 15) / 16;
    }
    for (int i = count; i <= kMaxFused; i++) a.rb_start[i] = nrb;
    a.count = count;
    a.x = x;
    a.in_scale = in_scale;
    a.in_scale_dev = in_scale_dev;
    a.cols = cols;
    a.groups = cols / kGroup;
    const int grid = sms < kMaxCtas ? sms : kMaxCtas;
    a.part_q = nrb / grid;
    a.part_r = nrb % grid;
    a.gpw = (a.groups + kWarps - 1) / kWarps;
    // shared memory: digit staging (512 B per group) | group factors | partial sums | rings
    size_t off = (mode == kI8) ? 0 : (size_t)kWarps * a.gpw * 512;
    a.off_xfac = (int)off;
    off += (size_t)kWarps * a.gpw * sizeof(float);
    off = (off + 15) & ~(size_t)15;
    a.off_part = (int)off;
    off += (size_t)(a.part_q + 1) * kWarps * 32 * sizeof(float);
    off = (off + 15) & ~(size_t)15;
    a.off_ring = (int)off;
    // deeper ring while two CTAs still fit in one SM's shared memory
    const size_t budget = (size_t)110 * 1024;
    const bool deep = off + (size_t)kWarps * 8 * kTileBytes <= budget;
    off += (size_t)kWarps * (deep ? 8 : 4) * kTileBytes;
    if (off > 227 * 1024) return TLLM_ERR_SIZE;           // caller falls back to the general streaming kernel
    if (mode == kI8) return deep ? launch_cw_t<kI8, 8>(a, grid, off, stream) : launch_cw_t<kI8, 4>(a, grid, off, stream);
    return deep ? launch_cw_t<kF16B1, 8>(a, grid, off, stream) : launch_cw_t<kF16B1, 4>(a, grid, off, stream);
}

// Several matrices that share x and the column count (q/k/v; gate/up) in one launch when
// together they fill the SMs; otherwise one launch each.
// x is FP16 (xq == nullptr) or INT8 with its scale in device memory.
static int gemv_packed_multi_any(int count, const uint8_t* const* packed, half* const* y, const int* rows, int cols,
                                 const half* x, const int8_t* xq, const float* scale_dev, cudaStream_t stream)
{
    DeviceScratch* s = nullptr;
    int st = get_scratch(&s);
    if (st) return st;
    const bool i8 = (xq != nullptr);
    // Matrices that were packed back to back (every row count but the last a multiple of 16)
    // are one contiguous tile array: stream them as one matrix, outputs scattered per segment.
    if (count >= 2 && count <= TLLM_MAX_FUSED) {
        bool contiguous = true;
        SegY seg = {};
        seg.n = count;
        int total = 0;
        for (int i = 0; i < count; i++) {
            if (i + 1 < count)
                contiguous = contiguous && (rows[i] % 16 == 0) && (packed[i + 1] == packed[i] + packed_bytes(rows[i], cols));
            seg.rows[i] = rows[i];
            seg.y[i] = y[i];
            total += rows[i];
        }
        if (contiguous)
            return i8 ? launch_packed_once(packed[0], xq, nullptr, 1.0f, kI8, 1, total, cols, stream, scale_dev, nullptr, &seg)
                      : launch_packed_once(packed[0], x, nullptr, 1.0f, kF16B1, 1, total, cols, stream, nullptr, nullptr, &seg);
    }
    // One fused launch pays off when some matrix alone cannot fill the SMs with whole row
    // blocks (k and v of grouped-query attention); matrices that can are streamed one by
    // one by the general kernel, which is the faster of the two for them.
    int nrb = 0;
    bool small = false;
    for (int i = 0; i < count; i++) {
        nrb += (rows[i] + 15) / 16;
        small = small || !cw_eligible(s->sms, rows[i], cols);
    }
    if (small && count >= 2 && count <= kMaxFused && cw_eligible_rb(s->sms, nrb, cols)) {
        st = launch_cw_multi(count, packed, y, rows, i8 ? (const void*)xq : (const void*)x, 1.0f,
                             i8 ? kI8 : kF16B1, cols, s->sms, stream, scale_dev);
        if (st != TLLM_ERR_SIZE) return st;
    }
    for (int i = 0; i < count; i++) {
        st = i8 ? launch_packed_once(packed[i], xq, y[i], 1.0f, kI8, 1, rows[i], cols, stream, scale_dev)
                : launch_gemv_packed(packed[i], x, y[i], 1, rows[i], cols, stream);
        if (st) return st;
    }
    return TLLM_OK;
}

// Several matrices that share x and the column count (q/k/v; gate/up) in one launch when
// together they fill the SMs; otherwise one launch each.
int launch_gemv_packed_multi(int count, const uint8_t* const* packed, half* const* y, const int* rows, int cols,
                             const half* x, cudaStream_t stream)
{
    return gemv_packed_multi_any(count, packed, y, rows, cols, x, nullptr, nullptr, stream);
}

// The same for INT8 activations whose scale stays in device memory (written by the
// quantiser that ran before on the stream), so that no host read sits between the two.
int launch_gemv_int8_packed_multi(int count, const uint8_t* const* packed, half* const* y, const int* rows,
                                  int cols, const int8_t* xq, const float* scale_dev, cudaStream_t stream)
{
    return gemv_packed_multi_any(count, packed, y, rows, cols, nullptr, xq, scale_dev, stream);
}

// INT8 GEMV whose activation vector is made inside the kernel (stage_x_fused):
// y = W . quantise(rmsnorm(a (+ b)) * w) with the rounded sum a + b stored to res_out, or
// y = W . quantise(silu(a) * b) when w == nullptr.
int launch_gemv_int8_packed_norm(const uint8_t* packed, const half* a, const half* b, const half* w, half* res_out,
                                 float eps, half* y, int rows, int cols, cudaStream_t stream)
{
    const FusedX fx = {a, b, w, res_out, eps};
    return launch_packed_once(packed, nullptr, y, 1.0f, kI8Norm, 1, rows, cols, stream, nullptr, &fx);
}

int launch_gemv_int8_packed_silu(const uint8_t* packed, const half* gate, const half* up, half* y, int rows, int cols,
                                 cudaStream_t stream)
{
    const FusedX fx = {gate, up, nullptr, nullptr, 0.f};
    return launch_packed_once(packed, nullptr, y, 1.0f, kI8Silu, 1, rows, cols, stream, nullptr, &fx);
}

int launch_gemv_int8_packed_quant(const uint8_t* packed, const half* x, half* y, int rows, int cols, cudaStream_t stream)
{
    const FusedX fx = {x, nullptr, nullptr, nullptr, 0.f};
    return launch_packed_once(packed, nullptr, y, 1.0f, kI8Quant, 1, rows, cols, stream, nullptr, &fx);
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

// ---------------------------------------------------------------------------
// GEMV for callers that must not allocate
// ---------------------------------------------------------------------------
// Some hosts of this library cannot let it call cudaMalloc: an inference server that
// has handed all device memory to its own arena, code running inside a region where
// the allocator is forbidden (a real-time loop, a stream capture), or a process whose
// memory budget is audited up front.  For them the split-K combine scratch of the
// GEMV lives in this fixed array instead of a lazily allocated buffer.  Every GPU that
// loads the library carries these 82 KB until the process exits.
//   [0, 65536)        partial-sum records, kMaxCtas x 64 floats
//   [65536, 81920)    arrival counters, kNoAllocMaxRowBlocks ints
//   [81920, 81924)    device error flag
constexpr int kNoAllocMaxRows = 65536;
constexpr int kNoAllocMaxRowBlocks = kNoAllocMaxRows / 16;
constexpr size_t kNoAllocWsBytes = (size_t)kMaxCtas * 64 * sizeof(float);
constexpr size_t kNoAllocCounterBytes = (size_t)kNoAllocMaxRowBlocks * sizeof(int);
constexpr size_t kNoAllocBytes = kNoAllocWsBytes + kNoAllocCounterBytes + 256;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

struct NoAllocDevice {
    unsigned char* base = nullptr;   // device address of g_noalloc_scratch on this device
    int sms = 0;
};
static NoAllocDevice g_noalloc[64];

// One FP16 vector, prepared weights, no allocation of any kind.  The first call on a
// device looks up the device address of the scratch array (cudaGetSymbolAddress, with
// that device current) and raises the kernel's shared-memory limit; make that first
// call outside any stream capture.  All calls share the one scratch array, which
// keeps what the previous call left: the counters are cleared on `stream` before each
// launch, and two calls whose kernels overlap on the GPU (different streams) race.
int launch_gemv_packed_noalloc(const uint8_t* packed, const half* x, half* y, int rows, int cols,
                               cudaStream_t stream)
{
    if (rows > kNoAllocMaxRows)
        return fail(TLLM_ERR_SIZE, "rows=%d exceeds the no-allocation variant's maximum of %d", rows, kNoAllocMaxRows);
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(TLLM_ERR_DEVICE, "no usable current device");
    NoAllocDevice& nd = g_noalloc[dev];
    if (!nd.base) {
        // In host code the array's name is only a handle; the kernel needs the address
        // the array has on THIS device.
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            return fail(TLLM_ERR_LAUNCH, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
        }
        if (cudaDeviceGetAttribute(&nd.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || nd.sms < 1)
            return fail(TLLM_ERR_DEVICE, "cannot read the SM count of device %d", dev);
        nd.base = static_cast<unsigned char*>(p);
    }
    GemvArgs a = {};
    a.packed = packed;
    a.x = x;
    a.y = y;
    a.in_scale = 1.0f;
    a.rows = rows;
    a.cols = cols;
    a.groups = cols / kGroup;
    a.batch = 1;
    const int nrb = (rows + 15) / 16;
    if ((long long)nrb * a.groups >= (1ll << 26))
        return fail(TLLM_ERR_SIZE, "rows=%d cols=%d: more than 2^26 tiles", rows, cols);
    const int tiles = nrb * a.groups;
    int grid = nd.sms < kMaxCtas ? nd.sms : kMaxCtas;
    const int per_cta_rb = (nrb + grid - 1) / grid;
    a.aligned = (nrb >= grid && (double)nrb / ((double)per_cta_rb * grid) >= 0.8) ? 1 : 0;
    // Fewer row blocks than SMs and short rows (one ring slot per warp at most): such a
    // matrix is a few hundred KB, latency-bound, and the cross-CTA combine would cost more
    // than the idle SMs; one CTA per row block.
    if (nrb < grid && a.groups <= kWarps * kSlotTiles) a.aligned = 1;
    // The same holds with a few more row blocks than SMs when a CTA's share is still at most
    // one ring slot per warp (q|k|v of a small model: 192 row blocks of 16 tiles).
    if (per_cta_rb * a.groups <= kWarps * kSlotTiles) a.aligned = 1;
    const int items = a.aligned ? nrb : tiles;
    if (items < grid) grid = items;
    a.part_q = items / grid;
    a.part_r = items % grid;
    a.late_release = release_rule(rows, cols);
    a.ws = reinterpret_cast<float*>(nd.base);
    a.counters = reinterpret_cast<int*>(nd.base + kNoAllocWsBytes);
    a.err = reinterpret_cast<int*>(nd.base + kNoAllocWsBytes + kNoAllocCounterBytes);
    size_t off = ((size_t)a.groups * 2 * 16 * 16 + 15) & ~(size_t)15;
    a.off_xfac = (int)off;
    off += (size_t)2 * a.groups * sizeof(float);
    off = (off + 15) & ~(size_t)15;
    a.off_part = (int)off;
    const int max_rb_per_cta = a.aligned ? (a.part_q + 1) : ((a.part_q + 1 + a.groups - 1) / a.groups + 1);
    off += (size_t)(max_rb_per_cta + kWarps) * 32 * sizeof(float);
    off = (off + 15) & ~(size_t)15;
    a.off_ring = (int)off;
    off += (size_t)kWarps * kRing * kSlotBytes;
    a.off_bar = (int)off;
    off += (size_t)kWarps * kRing * 8;
    if (off > 227 * 1024)
        return fail(TLLM_ERR_SIZE, "cols=%d needs %zu bytes of shared memory (limit 232448)", cols, off);
    // the counters must start at zero; a call that was cut short may have left some set
    if (cudaMemsetAsync(a.counters, 0, (size_t)nrb * sizeof(int), stream) != cudaSuccess) {
        cudaGetLastError();
        return fail(TLLM_ERR_LAUNCH, "clearing the scratch counters failed");
    }
    return launch_mode<kF16B1>(a, grid, off, stream, nullptr);
}

// Row-parallel GEMV with the all-reduce over peer memory fused into its epilogue.
int launch_gemv_packed_allreduce(const uint8_t* packed, const half* x, half* y, int rows, int cols, int rank,
                                 int world, void* const* peer_recv, void* epoch_local, int rows_max,
                                 cudaStream_t stream)
{
    DeviceScratch* s = nullptr;
    int st = get_scratch(&s);
    if (st) return st;
    if (world < 2 || world > kMaxPeers || rank < 0 || rank >= world)
        return fail(TLLM_ERR_SHAPE, "rank %d / world %d outside 2..%d ranks", rank, world, kMaxPeers);
    if (rows > rows_max) return fail(TLLM_ERR_SIZE, "rows=%d exceeds the receive buffers (%d rows)", rows, rows_max);
    GemvArgs a = {};
    a.packed = packed;
    a.x = x;
    a.y = y;
    a.in_scale = 1.0f;
    a.rows = rows;
    a.cols = cols;
    a.groups = cols / kGroup;
    a.batch = 1;
    const int nrb = (rows + 15) / 16;
    const int grid = s->sms < kMaxCtas ? s->sms : kMaxCtas;
    const int per_cta_rb = (nrb + grid - 1) / grid;
    if (nrb < grid || (double)nrb / ((double)per_cta_rb * grid) < 0.8)
        return fail(TLLM_ERR_SHAPE, "rows=%d: the fused all-reduce needs at least one 16-row block per SM", rows);
    a.aligned = 1;
    a.part_q = nrb / grid;
    a.part_r = nrb % grid;
    a.ws = s->ws;                       // unused in the aligned split
    a.counters = s->counters;
    a.err = s->misc + 1;
    a.ar_world = world;
    a.ar_rank = rank;
    a.ar_rows_max = rows_max;
    for (int d = 0; d < world; d++) a.ar_recv[d] = static_cast<uint2*>(peer_recv[d]);
    a.ar_epoch = static_cast<unsigned*>(epoch_local);
    size_t off = ((size_t)a.groups * 2 * 16 * 16 + 15) & ~(size_t)15;
    a.off_xfac = (int)off;
    off += (size_t)2 * a.groups * sizeof(float);
    off = (off + 15) & ~(size_t)15;
    a.off_part = (int)off;
    off += (size_t)(a.part_q + 1 + kWarps) * 32 * sizeof(float);
    off = (off + 15) & ~(size_t)15;
    a.off_ring = (int)off;
    off += (size_t)kWarps * kRing * kSlotBytes;
    a.off_bar = (int)off;
    off += (size_t)kWarps * kRing * 8;
    if (off > 227 * 1024) return fail(TLLM_ERR_SHAPE, "cols=%d needs %zu bytes of shared memory", cols, off);
    return launch_mode<kF16B1>(a, grid, off, stream, s);
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

// Device error flag of the current device (nullptr if the scratch cannot be set up).
int* device_error_flag()
{
    DeviceScratch* s = nullptr;
    if (get_scratch(&s) != TLLM_OK) return nullptr;
    return s->misc + 1;
}

// Synchronises `stream`, then reports and clears the device error flag.
int device_error_check(cudaStream_t stream)
{
    DeviceScratch* s = nullptr;
    int st = get_scratch(&s);
    if (st) return st;
    if (cudaStreamSynchronize(stream) != cudaSuccess)
        return fail(TLLM_ERR_LAUNCH, "stream sync: %s", cudaGetErrorString(cudaGetLastError()));
    int flag = 0;
    if (cudaMemcpy(&flag, s->misc + 1, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
        return fail(TLLM_ERR_LAUNCH, "error flag read: %s", cudaGetErrorString(cudaGetLastError()));
    if (flag != 0) {
        cudaMemset(s->misc + 1, 0, sizeof(int));
        return fail(flag, "a kernel reported status %d (bounded wait expired)", flag);
    }
    return TLLM_OK;
}

int weight_register(const void* nz, const uint8_t* packed, int rows, int cols)
{
    std::lock_guard<std::mutex> lk(g_reg_mu);
    g_registry[nz] = Registered{packed, rows, cols};
    return TLLM_OK;
}

#ifdef TLLM_PROFILE_PHASES
extern "C" int tllm_b200_debug_phases(unsigned long long* host_out, int n)
{
    return (int)cudaMemcpyFromSymbol(host_out, g_phase_ns, sizeof(unsigned long long) * n);
}
#endif

int weight_unregister(const void* nz)
{
    std::lock_guard<std::mutex> lk(g_reg_mu);
    g_registry.erase(nz);
    return TLLM_OK;
}

}  // namespace tllm

TL_DUMP(tllm_b200_debug_timeline_gemv)
