// Streaming ternary GEMV on the packed layout (packed_layout.cuh), sm_100a.
//
// The GEMV is HBM-bound: 2.125 bits per weight must stream at several TB/s, which
// leaves about 1.5 issue slots per weight per lane.  A masked add per weight on the
// CUDA cores costs 3-5, so the +x/-x/0 selection runs on the tensor cores instead.
// Weights are stored as 2-bit offset codes c = t + 1, sixteen to a word, arranged so
// that ONE logic instruction, `word & (0x03030303 << 2f)`, is an A-operand register of
// mma.sync.m16n8k32 (unsigned bytes c * 4^f for rows 16f..16f+15 of a 64-row
// super-tile).  The B operand carries the activations; integer MMA keeps every group
// sum exact; sum(t*x) = sum(c*x) - sum(x) with sum(x) made once per group when the
// activations are staged; the factor 4^f is divided out in FP32 with the scale.
//
//   FP16 activations: each scale group of 128 activations is converted once per CTA to
//   block fixed point, q = rint(x * 2^(22-e)) with 2^e > max|x| of the group, stored
//   as three BALANCED signed byte digits, q = d0 + 256*d1 + 65536*d2 with d in
//   [-128,127] (the bytes of q + 0x808080, each xor 0x80).  A vector occupies three B
//   columns [d0 d1 d2]; up to two vectors share one MMA (columns 0-2 and 4-6), up to
//   four take two MMAs per operand register.  Every digit sum is exact in INT32 and is
//   converted to FP32 once per group and row.  Rounding x to 23 bits below the group
//   maximum is at the level of FP32 accumulation rounding itself.  A group that holds a
//   NaN or an infinity makes its outputs NaN, as FP32 accumulation of x would.
//   INT8 activations (ternary_gemv_int8 semantics): B is the int8 vector as is.
//
// Work decomposition: the matrix is a linear array of super-tiles (64 rows x one scale
// group, 2176 bytes; row-block major).  They are dealt to CTAs (one per SM) and, inside
// a CTA, to 16 warps in contiguous, equal ranges, so K is split wherever rows alone
// would not balance 148 SMs.  Weights arrive through ONE ring of R slots per CTA
// (16-byte cp.async copies issued by all lanes of a warp, completion counted on one
// mbarrier per slot, a super-tile per slot -- measured on this part, a ring fed by
// cp.async.bulk tops out near 4 TB/s over the whole GPU whatever its depth, while
// per-thread loads reach the full HBM rate): the j-th super-tile
// of warp w has sequence number u = 16j + w and uses slot u mod R, so the ring is
// shared evenly whatever R is, R is simply what the shared-memory budget allows (two
// CTAs per SM: one computing, the next launch prefetching), and the first R are
// requested at kernel start.  The warp that finishes sequence number u refills its
// slot with u + R and publishes the slot's new use number in shared memory first: the
// consumer of u + R (another warp) looks at that number before it waits on the slot's
// mbarrier, because a parity wait on a barrier that is still one phase behind would
// return at once.  Partial sums of a 64-row block are combined in a fixed order:
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

constexpr int kWarpsLog2 = 4;
constexpr int kWarps = 1 << kWarpsLog2;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxSlots = 100;                        // ring slots per CTA, upper bound
constexpr int kTickets = 16;                          // independent scratch regions
constexpr int kMaxCtas = 256;
constexpr int kMaxVec = 4;                            // vectors per weight pass
constexpr int kRecFloats = kStRows * kMaxVec;         // one partial record: 64 rows x 4 vectors
constexpr int kMaxPeers = TLLM_MAX_PEERS;
// Dynamic shared memory of one CTA when two are to share an SM (228 KB per SM, 1 KB
// reserved per resident CTA).
#ifndef TLLM_GEMV_CORESIDENT_BYTES
#define TLLM_GEMV_CORESIDENT_BYTES (112 * 1024)
#endif
constexpr size_t kCoResidentBytes = TLLM_GEMV_CORESIDENT_BYTES;
constexpr size_t kMaxSmemBytes = 226 * 1024;      // dynamic part; the kernel also has a few static bytes
// L2 prefetch at kernel start of what a warp will stream beyond its first ring fill, in bytes
// per warp (0 = off).  The fill itself is bounded by shared memory; this lets the HBM stream
// of a launch go on into the 126 MB L2 while the launch still waits for the kernel before it.
#ifndef TLLM_GEMV_L2_PREFETCH_BYTES
#define TLLM_GEMV_L2_PREFETCH_BYTES 0
#endif
constexpr int kL2PrefetchSt = TLLM_GEMV_L2_PREFETCH_BYTES / kStBytes;

// kI8Norm / kI8Silu / kI8Quant: INT8 arithmetic like kI8, but the activation vector is
// produced inside the kernel's staging phase from FP16 inputs (stage_x_fused below).
enum Mode { kF16 = 0, kI8 = 2, kI8Norm = 3, kI8Silu = 4, kI8Quant = 5 };

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
    int rows, cols, groups; // groups = cols / 128 = super-tiles per row block
    int batch;              // vectors handled by this launch (1..4, FP16 modes)
    int part_q, part_r;     // items = gridDim.x * part_q + part_r; CTA c owns q (+1 if c < r) items
    int aligned;            // 1: items are whole row blocks (no block spans two CTAs); 0: items are super-tiles
    int late_release;       // 1: the next kernel in the stream is released after this kernel's own dependency
                            //    wait instead of at its start (see release_rule)
    int ring_slots;         // R
    int l2_prefetch;        // 1: a warp asks for (part of) its super-tiles beyond the first ring fill to be
                            //    brought into L2 at kernel start
    int x_local;            // FP16 modes, CTAs with fewer super-tiles than a row has groups: a CTA stages only
                            // the groups it walks (a cyclic run starting at its first super-tile's group)
    uint2* ws;              // [gridDim.x][2][ws_stride / 2] partial records {value, flag} of this ticket,
                            // all zero between launches
    int ws_stride;          // words per CTA in ws (two records)
    int* err;               // device error flag (0 = none)
    // shared memory carve-up (byte offsets); the staged activations start at 0
    int off_xcst, off_part, off_ring, off_bar, off_gen;
    // Fused all-reduce over peer memory (row-parallel shards of a tensor-parallel layer);
    // ar_world == 0 switches it off.  Every rank runs the same launch on its own shard.
    int ar_world, ar_rank, ar_rows_max;
    uint2* ar_recv[kMaxPeers];        // rank d's receive buffer  {value, launch number} [2][world][ar_rows_max]
    unsigned* ar_epoch;               // this rank's launch counters, uint [kMaxCtas]
    // Optional time stamps of the fused all-reduce (nullptr = off): CTA 0 writes, for launch
    // number e, the %globaltimer values {kernel entry, dependency wait over, partial sums ready,
    // peer stores issued, all ranks' words seen} to ar_trace[(e % ar_trace_cap) * 8 ..].
    unsigned long long* ar_trace;
    int ar_trace_cap;
};

// When a launch releases the next kernel of the stream.  Released at its start, the next
// kernel (and, through it, the one after) becomes resident while this one still runs and
// prefetches its own weights: a long stream of large matrices gains from that depth.  A small
// matrix lives on latencies, and the prefetch traffic of kernels two launches ahead queues in
// front of its activation loads and its final stores; such a launch releases its successor only
// after its own dependency wait, which bounds the look-ahead to one kernel.
#ifndef TLLM_LATE_RELEASE_BYTES
#define TLLM_LATE_RELEASE_BYTES (10u << 20)
#endif
static inline int release_rule(int rows, int cols)
{
    const size_t bytes = packed_bytes(rows, cols);
    return bytes <= (size_t)TLLM_LATE_RELEASE_BYTES ? 1 : 0;
}

// Diagnostic build only (python -m ternary_llm_b200.build --timeline, which defines
// TLLM_TIMELINE and writes libtllm_b200_timeline.so): thread 0 of every CTA of every GEMV launch
// records the GPU's nanosecond timer at seven points -- kernel entry, first ring fill issued,
// stream-order wait over, activations staged, last super-tile done, partial sums exchanged
// inside the CTA, outputs written -- into a ring of the last 8 launches, read back by
// tllm_b200_timeline_read.  The shipped library contains none of this.
#ifdef TLLM_TIMELINE
__device__ unsigned long long g_tl[8][kMaxCtas][8];
__device__ unsigned g_tl_cnt[kMaxCtas];
#define TL_BEGIN() unsigned tl_slot = 0; if (threadIdx.x == 0) tl_slot = g_tl_cnt[blockIdx.x]++ & 7u
#define TL(k) do { if (threadIdx.x == 0) g_tl[tl_slot][blockIdx.x][k] = globaltimer(); } while (0)
#else
#define TL_BEGIN()
#define TL(k)
#endif

// ---- PTX helpers ------------------------------------------------------------
__device__ __forceinline__ unsigned long long globaltimer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
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
// One super-tile global -> shared by the 32 lanes of a warp: 136 copies of 16 bytes (lanes 0..7
// issue a fifth one), then each lane makes the slot's mbarrier count its copies: the barrier
// (initialised to 32 arrivals) completes its phase when every lane's copies have landed.
__device__ __forceinline__ void fill_slot(uint32_t dst, const uint8_t* src, uint32_t bar, int lane)
{
#pragma unroll
    for (int i = 0; i < 4; i++)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                     ::"r"(dst + (uint32_t)(i * 32 + lane) * 16u), "l"(src + (size_t)(i * 32 + lane) * 16) : "memory");
    if (lane < kStBytes / 16 - 128)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                     ::"r"(dst + (uint32_t)(128 + lane) * 16u), "l"(src + (size_t)(128 + lane) * 16) : "memory");
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// D = A.B (+ D unless FIRST), A unsigned bytes (offset codes), B signed bytes.  The zero
// accumulator of the first step is passed as immediates so that no register is cleared.
template <bool FIRST>
__device__ __forceinline__ void imma(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                     uint32_t b0, uint32_t b1)
{
    if (FIRST)
        asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    else
        asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
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
// The n super-tiles of a CTA over its warps: warp w owns [w*n/kWarps, (w+1)*n/kWarps).
__device__ __forceinline__ int warp_start(int w, int n) { return (w * n) >> kWarpsLog2; }
__device__ __forceinline__ int warp_of(int i, int n) { return (int)((unsigned)((i + 1) * kWarps - 1) / (unsigned)n); }

// ---------------------------------------------------------------------------
// Activation staging
// ---------------------------------------------------------------------------
// Shared-memory layout of the staged activations, FP16 modes.  NB = MMA column blocks
// (n8) per operand register, NV = vectors per block (1 or 2).  Vector v lives in block
// v / NV... precisely: block beta = v >> 1 when NV == 2 (beta = 0 when NV == 1), column
// group vl = v & 1, so that the digit d of vector v is B column 4*vl + d of block beta.
//   xdig : uint4 [groups][2 step pairs][NB][NV*3 columns][4 lanes t]
//          the four words of an entry are (b0,b1) of k32 step 2p and (b0,b1) of step 2p+1 of
//          MMA lane (column, t), so one 128-bit shared load feeds two k32 steps;
//   xcst : uint4 [groups][NB*NV]  = {f, S01, 65536 f, S2}: f = 2^(e-22) of the group (NaN for a
//          group that holds a non-finite value), S01 = sum(d0 + 256 d1), S2 = sum(d2).
// The digit word of four consecutive activations: byte c of q + 0x808080, xor 0x80.
__device__ __forceinline__ void quad_digits(uint32_t q0, uint32_t q1, uint32_t q2, uint32_t q3,
                                            uint32_t& w0, uint32_t& w1, uint32_t& w2)
{
    const uint32_t u = __byte_perm(q0, q1, 0x5140), v = __byte_perm(q2, q3, 0x5140);
    const uint32_t r = __byte_perm(q0, q1, 0x0062), s = __byte_perm(q2, q3, 0x0062);
    w0 = __byte_perm(u, v, 0x5410) ^ 0x80808080u;
    w1 = __byte_perm(u, v, 0x7632) ^ 0x80808080u;
    w2 = __byte_perm(r, s, 0x5410) ^ 0x80808080u;
}

// Each thread converts 8 consecutive activations (one 128-bit load); the 16 lanes of a
// half-warp cover one scale group and agree on its exponent and sums with shuffles.
// The groups staged are the cyclic run g0, g0+1, ... (mod groups) of length gcount; staged
// group number i of that run is stored at index i (gcount == groups, g0 == 0: all of them).
template <int NB, int NV>
__device__ __forceinline__ void stage_x_f16(const half* __restrict__ x, int cols, int groups, int batch,
                                            uint32_t* xdig, uint4* xcst, int tid, int g0, int gcount)
{
    constexpr int NVT = NB * NV;
    const int per_vec = gcount << 4;               // 8-element items per vector (16 per group)
    const int items = per_vec * batch;
    const int l16 = tid & 15;
    // vectors of the last block that do not exist: their constants are zero, so whatever the
    // MMA makes of their (unwritten) digit columns never reaches a finite-times-NaN product
    for (int i = tid; i < gcount * (NVT - batch); i += kThreads) {
        const int g = i / (NVT - batch), v = batch + i % (NVT - batch);
        xcst[g * NVT + v] = make_uint4(0u, 0u, 0u, 0u);
    }
    for (int base = 0; base < items; base += kThreads) {
        const int item = base + tid;
        const bool valid = item < items;           // uniform per half-warp
        const int ic = valid ? item : 0;
        const int b = (int)((unsigned)ic / (unsigned)per_vec);
        const int el = ic - b * per_vec;           // item index inside the staged run
        const int g = el >> 4;                     // staged group number
        int gg = g0 + g;                           // its group in the vector
        if (gg >= groups) gg -= groups;
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + (size_t)b * cols) + (gg << 4) + (el & 15));
        float f[8];
        {
            const float2 f0 = __half22float2(*reinterpret_cast<const half2*>(&raw.x));
            const float2 f1 = __half22float2(*reinterpret_cast<const half2*>(&raw.y));
            const float2 f2 = __half22float2(*reinterpret_cast<const half2*>(&raw.z));
            const float2 f3 = __half22float2(*reinterpret_cast<const half2*>(&raw.w));
            f[0] = f0.x; f[1] = f0.y; f[2] = f1.x; f[3] = f1.y;
            f[4] = f2.x; f[5] = f2.y; f[6] = f3.x; f[7] = f3.y;
        }
        // largest magnitude as a bit pattern: orders finite values, infinities and NaNs alike
        uint32_t mb = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) mb = max(mb, __float_as_uint(f[i]) & 0x7fffffffu);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, o));
        const bool finite = mb < 0x7f800000u;
        // 2^e > max|x|; FP16 inputs keep e within [-23, 16]
        const int e = max((int)(mb >> 23) - 126, -24);
        const bool live = finite && mb != 0u;
        const float up = live ? __uint_as_float((uint32_t)(22 - e + 127) << 23) : 0.f;
        const float dn = finite ? (mb != 0u ? __uint_as_float((uint32_t)(e - 22 + 127) << 23) : 0.f)
                                : __uint_as_float(0x7fc00000u);
        uint32_t q[8];
        int sq = 0, s2 = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int qi = live ? __float2int_rn(f[i] * up) : 0;
            q[i] = (uint32_t)(qi + 0x808080);
            sq += qi;
            s2 += (int)((q[i] >> 16) & 0xffu) - 128;
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            sq += __shfl_xor_sync(0xffffffffu, sq, o);
            s2 += __shfl_xor_sync(0xffffffffu, s2, o);
        }
        uint32_t w[2][3];
        quad_digits(q[0], q[1], q[2], q[3], w[0][0], w[0][1], w[0][2]);
        quad_digits(q[4], q[5], q[6], q[7], w[1][0], w[1][1], w[1][2]);
        if (valid) {
            // elements 8*l16 .. 8*l16+7 of the group: k32 step m = l16 / 4, half j2 = (l16 / 2) & 1,
            // MMA lanes t = 2*(l16 & 1) and the next one
            const int m = l16 >> 2, j2 = (l16 >> 1) & 1, t0 = 2 * (l16 & 1);
            const int beta = (NV == 2) ? (b >> 1) : 0, vl = (NV == 2) ? (b & 1) : 0;
            uint32_t* p = xdig + ((((g * 2 + (m >> 1)) * NB + beta) * (NV * 3) + vl * 3) * 4 + t0) * 4 + (m & 1) * 2 + j2;
#pragma unroll
            for (int h = 0; h < 2; h++)             // second quad: next lane t
#pragma unroll
                for (int d = 0; d < 3; d++) p[(d * 4 + h) * 4] = w[h][d];
            if (l16 == 0) {
                const float dn16 = dn * 65536.0f;
                xcst[g * NVT + b] = make_uint4(__float_as_uint(dn), (uint32_t)(sq - 65536 * s2),
                                               __float_as_uint(dn16), (uint32_t)s2);
            }
        }
    }
}

// INT8 activations in shared memory are permuted so that the four B words a lane needs for
// two k32 steps are one 128-bit entry: uint4 [groups][2 step pairs][4 lanes t], words
// (b0,b1) of step 2p and (b0,b1) of step 2p+1.  Original word w of the vector (four
// consecutive activations) goes to this 32-bit slot.
__device__ __forceinline__ int int8_word_slot(int w)
{
    const int g = w >> 5, r = w & 31;
    const int m = r >> 3, j2 = (r >> 2) & 1, t = r & 3;
    return (g << 5) + ((((m >> 1) << 2) + t) << 2) + ((m & 1) << 1) + j2;
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

// Sum of the four signed bytes of a word.
__device__ __forceinline__ int byte_sum(uint32_t w) { return __dp4a((int)w, 0x01010101, 0); }

// INT8 vector from global memory: permuted copy plus the per-group sums sx[groups].
__device__ __forceinline__ void stage_x_i8(const int8_t* __restrict__ x, int cols, uint32_t* xq, int* sx, int tid)
{
    const int n16 = cols >> 4;                     // 16-byte items (8 per group)
    const uint4* src = reinterpret_cast<const uint4*>(x);
    for (int base = 0; base < n16; base += kThreads) {
        const int i = base + tid;
        const bool valid = i < n16;                // uniform per 8 lanes
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (valid) v = __ldg(src + i);
        int s = byte_sum(v.x) + byte_sum(v.y) + byte_sum(v.z) + byte_sum(v.w);
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (valid) {
            // words 4i .. 4i+3 share the k32 step and the half, their lanes are t = 0..3
            const int s0 = int8_word_slot(4 * i);
            xq[s0] = v.x;
            xq[s0 + 4] = v.y;
            xq[s0 + 8] = v.z;
            xq[s0 + 12] = v.w;
            if ((i & 7) == 0) sx[i >> 3] = s;
        }
    }
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
// Returns the activation scale.  tmp: half [cols]; red: 33 floats; sx: int [groups].
template <int MODE>
__device__ __forceinline__ float stage_x_fused(const GemvArgs& a, uint32_t* xq, int* sx, half* tmp, float* red, int tid)
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
    for (int base = 0; base < n8; base += kThreads) {
        const int i = base + tid;
        const bool valid = i < n8;                 // uniform per half-warp (n8 is a multiple of 16)
        uint4 v4 = make_uint4(0u, 0u, 0u, 0u);
        if (valid) v4 = *(reinterpret_cast<const uint4*>(tmp) + i);
        const half* vh = reinterpret_cast<const half*>(&v4);
        uint32_t w[2];
        int s = 0;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            uint32_t acc = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int qv = max(-127, min(127, __float2int_rn(__half2float(vh[h * 4 + j]) * inv)));
                acc |= (uint32_t)(qv & 0xff) << (8 * j);
                s += qv;
            }
            w[h] = acc;
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (valid) {
            xq[int8_word_slot(2 * i)] = w[0];
            xq[int8_word_slot(2 * i + 1)] = w[1];
            if ((i & 15) == 0) sx[i >> 4] = s;
        }
    }
    return (absmax > 0.f) ? (absmax / 127.0f) : 1.0f;
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
template <int MODE, int NB, int NV, bool AR>
__global__ void __launch_bounds__(kThreads, 2) gemv_packed_kernel(const GemvArgs a)
{
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr bool FUSEDX = (MODE == kI8Norm || MODE == kI8Silu || MODE == kI8Quant);
    constexpr bool I8 = (MODE == kI8 || FUSEDX);
    constexpr int NVT = NB * NV;                  // vectors per weight pass
    static_assert(!I8 || (NB == 1 && NV == 1), "INT8 modes carry one vector");

    if (!a.late_release) asm volatile("griddepcontrol.launch_dependents;");

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // the fused all-reduce is an instantiation of its own (one FP16 vector only)
    constexpr bool kAr = AR;
    static_assert(!AR || (MODE == kF16 && NB == 1 && NV == 1), "the fused all-reduce carries one FP16 vector");
    __shared__ unsigned long long ts[5];     // time stamps of a traced all-reduce launch (thread 0 of CTA 0)
    const bool tracing = kAr && (a.ar_trace != nullptr) && blockIdx.x == 0 && tid == 0;
    if (tracing) ts[0] = globaltimer();
    TL_BEGIN();
    TL(0);
    const int G = a.groups, R = a.ring_slots;
    const int per = a.aligned ? G : 1;                                     // super-tiles per partition item
    const int t0 = part_start(blockIdx.x, a.part_q, a.part_r) * per;      // first super-tile of this CTA
    const int n = (a.part_q + ((int)blockIdx.x < a.part_r ? 1 : 0)) * per; // super-tiles of this CTA
    const int rb_first = (int)((unsigned)t0 / (unsigned)G);
    const int rb_last = (int)((unsigned)(t0 + n - 1) / (unsigned)G);

    uint32_t* xstage = reinterpret_cast<uint32_t*>(smem);              // digits, or the int8 vector
    uint4* xcst = reinterpret_cast<uint4*>(smem + a.off_xcst);         // FP16 modes: group constants
    int* sx = reinterpret_cast<int*>(smem + a.off_xcst);               // INT8 modes: group sums
    float* part = reinterpret_cast<float*>(smem + a.off_part);         // [segment][64 rows][NVT]
    const uint32_t ring = smem_addr(smem + a.off_ring);
    const uint8_t* ring_p = smem + a.off_ring;
    const uint32_t bar = smem_addr(smem + a.off_bar);
    volatile uint32_t* gen = reinterpret_cast<volatile uint32_t*>(smem + a.off_gen);   // use number of each slot

    // ---- this warp's super-tile range and the first ring fill ---------------------
    const int w0 = t0 + warp_start(warp, n), w1 = t0 + warp_start(warp + 1, n);
    const int nw = w1 - w0;                                  // may be 0 for tiny problems
    if (lane == 0) {
        for (int s = warp; s < R; s += kWarps) {
            mbar_init(bar + s * 8, 32);
            gen[s] = 0u;
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    {
        // sequence numbers 16j + warp < R go to slots of the same number
        int j = 0;
        for (int s = warp; s < R && j < nw; j++, s += kWarps)
            fill_slot(ring + s * kStBytes, a.packed + (size_t)(w0 + j) * kStBytes, bar + s * 8, lane);
        if (kL2PrefetchSt > 0 && a.l2_prefetch && j < nw && lane == 0) {
            const uint32_t bytes = (uint32_t)min(nw - j, kL2PrefetchSt) * kStBytes;
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;"
                         ::"l"(a.packed + (size_t)(w0 + j) * kStBytes), "r"(bytes) : "memory");
        }
    }
    __syncwarp();
    TL(1);

    // ---- everything below may depend on the previous kernel in the stream -------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (a.late_release) asm volatile("griddepcontrol.launch_dependents;");
    if (tracing) ts[1] = globaltimer();
    TL(2);
    // launch number of the fused all-reduce (written by this rank's previous such launch):
    // requested here so that the load's latency hides behind the staging
    unsigned ar_epoch_prev = 0;
    if (kAr && a.ar_world > 0) ar_epoch_prev = __ldcg(a.ar_epoch + blockIdx.x);

    float fused_scale = 1.0f;
    if (FUSEDX) {
        fused_scale = stage_x_fused<MODE>(a, xstage, sx, reinterpret_cast<half*>(smem + a.off_xtmp),
                                          reinterpret_cast<float*>(smem + a.off_xtmp + (size_t)a.cols * sizeof(half)), tid);
    } else if (I8) {
        stage_x_i8(reinterpret_cast<const int8_t*>(a.x), a.cols, xstage, sx, tid);
    } else {
        const int g0 = a.x_local ? (int)((unsigned)t0 % (unsigned)G) : 0;
        stage_x_f16<NB, NV>(reinterpret_cast<const half*>(a.x), a.cols, G, a.batch, xstage, xcst, tid, g0,
                            a.x_local ? n : G);
    }
    __syncthreads();
    TL(3);

    // ---- per-lane constants ------------------------------------------------------
    const int t = lane & 3, gq = lane >> 2;
    // FP16: this lane's accumulator columns 2t, 2t+1 are digits (0,1) of vector t/2 of the
    // block when t is even, digit 2 (and an unused column) when t is odd
    const int mulA = (t & 1) ? 0 : 256;
    // B operand entry of this lane: column gq -> (vector gq / 4 of the block, digit gq % 4);
    // lanes of columns that carry nothing read a neighbour's entry, their products are unused
    const int bcol = min(gq >> 2, NV - 1) * 3 + min(gq & 3, 2);
    const uint4* xb_lane = reinterpret_cast<const uint4*>(xstage) + (I8 ? t : bcol * 4 + t);
    constexpr int kXbStride = I8 ? 4 : NV * 12;                 // entries per (group, step pair, block)

    // ---- main loop: this warp's super-tiles, one ring slot each --------------------
    int rb = (int)((unsigned)w0 / (unsigned)G);
    int g = w0 - rb * G;
    int gx_local = w0 - t0;                  // FP16 modes with x_local: where group g's activations were staged
    int seg = (rb - rb_first) + warp;        // partial-sum slot: unique per (warp, row block), ascending
    float acc[NB][4][2];                     // [block][field f][row half h]: rows 16f + gq + 8h of row block rb
#pragma unroll
    for (int b = 0; b < NB; b++)
#pragma unroll
        for (int f = 0; f < 4; f++) acc[b][f][0] = acc[b][f][1] = 0.f;
    bool dirty = false, ok = true;

    auto flush = [&]() {
        float* pu = part + (size_t)seg * (kStRows * NVT);
#pragma unroll
        for (int b = 0; b < NB; b++)
#pragma unroll
            for (int f = 0; f < 4; f++)
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    float v = acc[b][f][h] * (1.0f / (float)(1 << (2 * f)));
                    if (!I8) v += __shfl_xor_sync(0xffffffffu, v, 1);   // lanes t, t^1: the digit halves of one vector
                    const int row = 16 * f + gq + 8 * h;
                    if (I8) {
                        if (t == 0) pu[row] = v;
                    } else if ((t & 1) == 0 && (t >> 1) < NV) {
                        pu[row * NVT + b * NV + (t >> 1)] = v;
                    }
                    acc[b][f][h] = 0.f;
                }
        dirty = false;
    };

    int slot = warp;
    uint32_t use = 0;                        // how often this slot has been filled before: sequence number / R
    for (int j = 0; j < nw; j++) {
        // the slot's barrier must have reached the phase of this use before its parity means
        // anything: the warp that emptied the slot publishes the use number when it refills it
        if (use > 0) {
            ok = false;
#pragma unroll 1
            for (int i = 0; i < (1 << 22); i++)
                if (gen[slot] >= use) {
                    ok = true;
                    break;
                }
            if (!ok) break;
        }
        ok = mbar_wait(bar + slot * 8, use & 1u);
        if (!ok) break;
        const uint8_t* tile = ring_p + (size_t)slot * kStBytes;
        const int gx = (!I8 && a.x_local) ? gx_local : g;
        const uint4* codes = reinterpret_cast<const uint4*>(tile) + lane;
        const uint4 s8 = *reinterpret_cast<const uint4*>(tile + kStCodeBytes + gq * 16);
#pragma unroll
        for (int b = 0; b < NB; b++) {
            int d[4][4];
            uint4 xb;
#pragma unroll
            for (int m = 0; m < 4; m++) {
                const uint4 wd = codes[m * 32];
                if ((m & 1) == 0) xb = xb_lane[((gx * 2 + (m >> 1)) * NB + b) * kXbStride];
                const uint32_t b0 = (m & 1) ? xb.z : xb.x, b1 = (m & 1) ? xb.w : xb.y;
#pragma unroll
                for (int f = 0; f < 4; f++) {
                    const uint32_t msk = 0x03030303u << (2 * f);
                    // words (h, j2) = (0,0) (0,1) (1,0) (1,1) are registers a0, a2, a1, a3
                    if (m == 0) imma<true>(d[f], wd.x & msk, wd.z & msk, wd.y & msk, wd.w & msk, b0, b1);
                    else imma<false>(d[f], wd.x & msk, wd.z & msk, wd.y & msk, wd.w & msk, b0, b1);
                }
            }
            // group epilogue: remove the code offset, apply scale and block exponent
            float fx;
            int soff;
            if (I8) {
                fx = 1.0f;
                soff = sx[gx];
            } else {
                const int v = min(b * NV + (t >> 1), NVT - 1);
                const uint2 c = reinterpret_cast<const uint2*>(xcst + gx * NVT + v)[t & 1];
                fx = __uint_as_float(c.x);
                soff = (int)c.y;
            }
            const uint32_t sw[4] = {s8.x, s8.y, s8.z, s8.w};
#pragma unroll
            for (int f = 0; f < 4; f++) {
                const float2 sc = __half22float2(*reinterpret_cast<const half2*>(&sw[f]));
                const int o = soff * (1 << (2 * f));
                const int p0 = I8 ? (d[f][0] - o) : (d[f][1] * mulA + d[f][0] - o);
                const int p1 = I8 ? (d[f][2] - o) : (d[f][3] * mulA + d[f][2] - o);
                acc[b][f][0] = fmaf((float)p0, sc.x * fx, acc[b][f][0]);
                acc[b][f][1] = fmaf((float)p1, sc.y * fx, acc[b][f][1]);
            }
        }
        dirty = true;
        // refill this slot with sequence number u + R (it belongs to warp (u + R) mod 16)
        __syncwarp();
        {
            const int u2 = j * kWarps + warp + R;
            const int w2 = u2 & (kWarps - 1), j2 = u2 >> kWarpsLog2;
            const int s2 = warp_start(w2, n);
            if (j2 < warp_start(w2 + 1, n) - s2) {
                if (lane == 0) gen[slot] = use + 1u;
                fill_slot(ring + slot * kStBytes, a.packed + (size_t)(t0 + s2 + j2) * kStBytes, bar + slot * 8, lane);
            }
        }
        slot += kWarps;
        if (slot >= R) {
            slot -= R;
            use++;
        }
        gx_local++;
        if (++g == G) {                      // row block finished (for this warp)
            flush();
            g = 0;
            rb++;
            seg++;
        }
    }
    if (dirty) flush();
    if (!ok && lane == 0) atomicExch(a.err, TLLM_ERR_TIMEOUT);
    TL(4);
    __syncthreads();
    TL(5);

    // ---- reduction: warps of this CTA, then CTAs, row block by row block -----------
    const int nb = I8 ? 1 : a.batch;
    const float oscale = FUSEDX ? fused_scale : (I8 ? (a.in_scale_dev ? __ldg(a.in_scale_dev) : a.in_scale) : 1.0f);
    constexpr int kRec = kStRows * NVT;      // floats of one row block's sums

    if (kAr && a.ar_world > 0) {
        // ---- fused all-reduce: my partial sums go straight into every rank's receive
        // buffer over NVLink as 8-byte {value, launch number} words -- the store of a word
        // is atomic, so the launch number doubles as the arrival flag and no fence or
        // separate flag round is needed.  Each CTA then polls (bounded) its OWN memory for
        // the other ranks' words of the same rows -- every rank runs this launch with the
        // same partition -- and adds the contributions in rank order.  Buffers alternate
        // with the launch parity, so a rank that runs one launch ahead never overwrites
        // words that are still being read.
        __shared__ int ar_abort;
        if (tid == 0) ar_abort = 0;
        if (tracing) ts[2] = globaltimer();
        const unsigned epoch = ar_epoch_prev + 1u;
        const unsigned epar = epoch & 1u;
        const size_t wslot = (size_t)(epar * a.ar_world + a.ar_rank) * a.ar_rows_max;
        for (int r_b = rb_first + warp; r_b <= rb_last; r_b += kWarps) {
            const int ta = max(t0, r_b * G), tb = min(t0 + n, (r_b + 1) * G);
            const int wa = warp_of(ta - t0, n), wb = warp_of(tb - 1 - t0, n);
            for (int idx = lane; idx < kStRows; idx += 32) {
                float s = 0.f;
                for (int w = wa; w <= wb; w++)
                    if (warp_start(w + 1, n) > warp_start(w, n)) s += part[(size_t)((r_b - rb_first) + w) * kRec + idx];
                const int r = r_b * kStRows + idx;
                if (r < a.rows) {
                    const uint2 word = make_uint2(__float_as_uint(s), epoch);
#pragma unroll
                    for (int dst_rank = 0; dst_rank < kMaxPeers; dst_rank++) {
                        if (dst_rank < a.ar_world) {
                            uint2* dst = a.ar_recv[dst_rank] + wslot + r;
                            asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(word.x), "r"(word.y) : "memory");
                        }
                    }
                }
            }
        }
        __syncthreads();                     // ar_abort initialised; all stores issued
        if (tracing) ts[3] = globaltimer();
        const int r_lo = rb_first * kStRows, r_hi = min(a.rows, (rb_last + 1) * kStRows);
        const uint2* recv = a.ar_recv[a.ar_rank] + (size_t)epar * a.ar_world * a.ar_rows_max;
        const unsigned all = (1u << a.ar_world) - 1u;
        bool ok_ar = true;
        for (int r = r_lo + tid; r < r_hi; r += kThreads) {
            // one look at ALL ranks' words per round (independent loads in flight together), then
            // only at the missing ones.  About half a second at most for the first wait that
            // expires; once one has, every later wait of this CTA gives up at its first look.
            uint32_t val[kMaxPeers];
            unsigned pending = all;
#pragma unroll 1
            for (int i = 0; i < (1 << 21) && pending; i++) {
                uint32_t tag[kMaxPeers];
#pragma unroll
                for (int d = 0; d < kMaxPeers; d++) {
                    tag[d] = 0;
                    if ((pending >> d) & 1u) {
                        const uint2* src = recv + (size_t)d * a.ar_rows_max + r;
                        asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(val[d]), "=r"(tag[d]) : "l"(src) : "memory");
                    }
                }
#pragma unroll
                for (int d = 0; d < kMaxPeers; d++)
                    if (((pending >> d) & 1u) && tag[d] == epoch) pending &= ~(1u << d);
                if (pending) {
                    if (*(volatile int*)&ar_abort) break;
                    __nanosleep(20);
                }
            }
            if (pending) {
                ok_ar = false;
                ar_abort = 1;
            }
            float v = 0.f;
#pragma unroll
            for (int d = 0; d < kMaxPeers; d++)
                if (d < a.ar_world) v += __uint_as_float(val[d]);      // rank order: the same sum on every rank
            a.y[r] = __float2half_rn(v);
        }
        if (!ok_ar) atomicExch(a.err, TLLM_ERR_TIMEOUT);
        __syncthreads();
        if (tid == 0) a.ar_epoch[blockIdx.x] = epoch;
        if (tracing) {
            ts[4] = globaltimer();
            unsigned long long* rec = a.ar_trace + (size_t)(epoch % (unsigned)a.ar_trace_cap) * 8;
#pragma unroll
            for (int i = 0; i < 5; i++) rec[i] = ts[i];
            rec[5] = epoch;
        }
        return;
    }

    uint2* myrec = a.ws + (size_t)blockIdx.x * a.ws_stride;
    const int rec1 = a.ws_stride >> 1;        // offset of a CTA's second record
    constexpr int kW = kRec / 32;             // words per lane in one record
    constexpr int kChunk = (kW >= 8) ? 1 : ((kW >= 4) ? 2 : 4);      // records polled together
    bool ok_c = true;
    for (int r_b = rb_first + warp; r_b <= rb_last; r_b += kWarps) {
        const int ta = max(t0, r_b * G), tb = min(t0 + n, (r_b + 1) * G);     // this CTA's super-tiles of the block
        const int wa = warp_of(ta - t0, n), wb = warp_of(tb - 1 - t0, n);
        const bool full = (tb - ta == G);
        float s[kW];
#pragma unroll
        for (int i = 0; i < kW; i++) {
            const int idx = lane + 32 * i;
            float v = 0.f;
            for (int w = wa; w <= wb; w++)
                if (warp_start(w + 1, n) > warp_start(w, n))       // warps without super-tiles wrote nothing
                    v += part[(size_t)((r_b - rb_first) + w) * kRec + idx];
            s[i] = v;
        }
        if (!full) {
            // This row block is shared with neighbouring CTAs (K is split across them).  All but
            // the last of them publish their sums and are done; the last gathers.
            const int c_a = part_of(r_b * G, a.part_q, a.part_r);
            const int c_b = part_of((r_b + 1) * G - 1, a.part_q, a.part_r);
            if ((int)blockIdx.x != c_b) {
                uint2* rec = myrec + ((r_b == rb_first) ? 0 : rec1);
#pragma unroll
                for (int i = 0; i < kW; i++)
                    asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1, %2};"
                                 ::"l"(rec + lane + 32 * i), "r"(__float_as_uint(s[i])), "r"(1u) : "memory");
                continue;
            }
            float tot[kW];
#pragma unroll
            for (int i = 0; i < kW; i++) tot[i] = 0.f;
            for (int c0 = c_a; c0 < c_b; c0 += kChunk) {
                uint2* rec[kChunk];
                uint32_t val[kChunk][kW];
                unsigned pending = 0;
#pragma unroll
                for (int cc = 0; cc < kChunk; cc++) {
                    const int c = min(c0 + cc, c_b - 1);
                    // record 0 of a CTA belongs to its first row block, record 1 to its last
                    const int c_rb = (int)((unsigned)part_start(c, a.part_q, a.part_r) / (unsigned)G);
                    rec[cc] = a.ws + (size_t)c * a.ws_stride + ((r_b == c_rb) ? 0 : rec1) + lane;
                    if (c0 + cc < c_b) pending |= ((1u << kW) - 1u) << (cc * kW);
                }
                // all words of the chunk are requested together, then only the missing ones; a
                // wait that expires (about half a second) ends every later wait of this CTA at once
#pragma unroll 1
                for (int it = 0; it < (1 << 21) && pending; it++) {
                    uint32_t v[kChunk][kW], f[kChunk][kW];
#pragma unroll
                    for (int cc = 0; cc < kChunk; cc++)
#pragma unroll
                        for (int i = 0; i < kW; i++) {
                            f[cc][i] = 0;
                            if ((pending >> (cc * kW + i)) & 1u)
                                asm volatile("ld.relaxed.gpu.global.v2.u32 {%0, %1}, [%2];"
                                             : "=r"(v[cc][i]), "=r"(f[cc][i]) : "l"(rec[cc] + 32 * i) : "memory");
                        }
#pragma unroll
                    for (int cc = 0; cc < kChunk; cc++)
#pragma unroll
                        for (int i = 0; i < kW; i++)
                            if (f[cc][i]) {
                                val[cc][i] = v[cc][i];
                                pending &= ~(1u << (cc * kW + i));
                            }
                    if (pending) {
                        if (!ok_c) break;
                        __nanosleep(20);
                    }
                }
                if (pending) ok_c = false;
#pragma unroll
                for (int cc = 0; cc < kChunk; cc++)
                    if (c0 + cc < c_b) {
#pragma unroll
                        for (int i = 0; i < kW; i++) {
                            tot[i] += __uint_as_float(val[cc][i]);
                            asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1, %1};"
                                         ::"l"(rec[cc] + 32 * i), "r"(0u) : "memory");
                        }
                    }
            }
#pragma unroll
            for (int i = 0; i < kW; i++) s[i] += tot[i];            // own part last: CTA order
        }
#pragma unroll
        for (int i = 0; i < kW; i++) {
            const int idx = lane + 32 * i;
            const int r = r_b * kStRows + idx / NVT, b = idx % NVT;
            if (r < a.rows && b < nb) *out_ptr(a, b, r) = __float2half_rn(s[i] * oscale);
        }
    }
    if (!ok_c) atomicExch(a.err, TLLM_ERR_TIMEOUT);
    TL(6);
}

// ---------------------------------------------------------------------------
// Repack: reference layout -> packed layout, and back
// ---------------------------------------------------------------------------
// one thread per code word of the packed matrix; the threads of words (m = 0, t = 0, j2 = 0)
// also write their rows' scales.  Counts sign bits that have no nonzero bit.
__global__ void repack_kernel(const uint32_t* __restrict__ nz, const uint32_t* __restrict__ sg,
                              const half* __restrict__ scales, uint8_t* __restrict__ packed,
                              int rows, int cols, int* __restrict__ noncanon)
{
    const int groups = cols / kGroup, wpr = cols / 32;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long nst = (long long)((rows + kStRows - 1) / kStRows) * groups;
    if (idx >= nst * 512) return;
    const long long st = idx >> 9;
    const int wi = (int)(idx & 511);
    const int m = wi >> 7, lane = (wi >> 2) & 31, i = wi & 3;
    const int gq = lane >> 2, t = lane & 3, h = i >> 1, j2 = i & 1;
    const int rb = (int)(st / groups), g = (int)(st % groups);
    const int bit0 = 16 * j2 + 4 * t;                       // first of this word's four bits in the mask word
    uint32_t word = 0, stray = 0;
    for (int f = 0; f < 4; f++) {
        const int r = rb * kStRows + 16 * f + gq + 8 * h;
        uint32_t a = 0, s = 0;
        if (r < rows) {
            a = nz[(size_t)r * wpr + g * 4 + m];
            s = sg[(size_t)r * wpr + g * 4 + m];
        }
        a = (a >> bit0) & 0xfu;
        s = (s >> bit0) & 0xfu;
        stray += __popc(s & ~a);
        for (int j = 0; j < 4; j++) {
            const uint32_t nzb = (a >> j) & 1u, sgb = (s >> j) & 1u;
            const uint32_t code = nzb ? (sgb ? 2u : 0u) : 1u;       // t + 1
            word |= code << (8 * j + 2 * f);
        }
    }
    reinterpret_cast<uint32_t*>(packed + (size_t)st * kStBytes)[wi] = word;
    if (stray) atomicAdd(noncanon, (int)stray);
    if (m == 0 && t == 0 && j2 == 0) {
        half* sp = reinterpret_cast<half*>(packed + (size_t)st * kStBytes + kStCodeBytes);
        for (int f = 0; f < 4; f++) {
            const int r64 = 16 * f + gq + 8 * h, r = rb * kStRows + r64;
            sp[st_scale_index(r64)] = (r < rows) ? scales[(size_t)r * groups + g] : __float2half(0.f);
        }
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
    const int g = wd / 4, m = wd % 4;          // mask word wd covers group columns 32m .. 32m+31 = k32 step m
    const uint8_t* tp = packed + ((size_t)(r / kStRows) * groups + g) * kStBytes;
    const uint32_t* cw = reinterpret_cast<const uint32_t*>(tp);
    const int r64 = r % kStRows;
    uint32_t a = 0, s = 0;
    for (int c = 0; c < 32; c++) {
        int word, shift;
        st_locate(r64, 32 * m + c, word, shift);
        const uint32_t code = (cw[word] >> shift) & 3u;
        if (code != 1u) a |= 1u << c;
        if (code == 2u) s |= 1u << c;
    }
    nz[idx] = a;
    sg[idx] = s;
    if (m == 0) scales[(size_t)r * groups + g] = reinterpret_cast<const half*>(tp + kStCodeBytes)[st_scale_index(r64)];
}

// ---------------------------------------------------------------------------
// Host side: scratch, registry, launch
// ---------------------------------------------------------------------------
constexpr int kMaxRowBlocks = 1 << 16;          // rows up to 4,194,304
struct DeviceScratch {
    uint2* ws = nullptr;       // [kTickets][kMaxCtas][2][kRecFloats] {value, flag}, all zero between launches
    int* misc = nullptr;       // [0] non-canonical bit counter of the last prepare, [1] device error flag
    int sms = 0;
    unsigned ticket = 0;
    bool ready = false;
};
static DeviceScratch g_scratch[64];
static std::mutex g_mu;

static int get_scratch(DeviceScratch** out)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(TLLM_ERR_DEVICE, "no usable current device");
    DeviceScratch& s = g_scratch[dev];
    std::lock_guard<std::mutex> lk(g_mu);
    if (!s.ready) {
        // First use on this device: allocate and zero the scratch.  Must not happen
        // inside a stream capture; make one call per device before capturing.
        cudaDeviceGetAttribute(&s.sms, cudaDevAttrMultiProcessorCount, dev);
        if (cudaMalloc(&s.ws, (size_t)kTickets * kMaxCtas * 2 * kRecFloats * sizeof(uint2)) != cudaSuccess ||
            cudaMalloc(&s.misc, 64) != cudaSuccess)
            return fail(TLLM_ERR_LAUNCH, "scratch allocation failed: %s", cudaGetErrorString(cudaGetLastError()));
        cudaMemset(s.ws, 0, (size_t)kTickets * kMaxCtas * 2 * kRecFloats * sizeof(uint2));
        cudaMemset(s.misc, 0, 64);
        cudaDeviceSynchronize();
        s.ready = true;
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
    return (size_t)((rows + kStRows - 1) / kStRows) * (size_t)(cols / kGroup) * kStBytes;
}

int packed_row_align() { return kStRows; }

// Partition of the matrix over CTAs and the shared-memory layout of one launch; the same for
// every entry point (regular, no-allocation, fused all-reduce), which differ only in where the
// cross-CTA scratch lives.  nvt = vectors per pass as instantiated (1, 2 or 4), nvx = vector
// columns stored per group (NB * NV * 3 digit columns), force_aligned: whole row blocks per
// CTA or fail (the fused all-reduce needs it).
static int plan_gemv(GemvArgs& a, int sms, int mode, int nvt, int max_ctas, bool force_aligned, int* grid_out,
                     size_t* smem_out)
{
    const int rows = a.rows, cols = a.cols;
    a.groups = cols / kGroup;
    const int nrb = (rows + kStRows - 1) / kStRows;
    if (nrb > kMaxRowBlocks) return fail(TLLM_ERR_SHAPE, "rows=%d exceeds %d", rows, kMaxRowBlocks * kStRows);
    if ((long long)nrb * a.groups >= (1ll << 26))
        return fail(TLLM_ERR_SHAPE, "rows=%d cols=%d: more than 2^26 super-tiles", rows, cols);
    const int tiles = nrb * a.groups;
    const int grid_max = sms < max_ctas ? sms : max_ctas;
    const bool fusedx = (mode == kI8Norm || mode == kI8Silu || mode == kI8Quant);
    const bool i8 = (mode == kI8 || fusedx);
    const int per_cta_rb = (nrb + grid_max - 1) / grid_max;

    // Shared-memory layout for one way of cutting the matrix: activations | group constants |
    // partial sums | (fused staging) | mbarriers | use numbers | ring.  Returns the bytes in
    // front of the ring.
    auto layout = [&](int aligned, int* grid, int* n_max_out) {
        a.aligned = aligned;
        const int items = aligned ? nrb : tiles;
        *grid = items < grid_max ? items : grid_max;
        a.part_q = items / *grid;
        a.part_r = items % *grid;
        const int n_max = (a.part_q + (a.part_r ? 1 : 0)) * (aligned ? a.groups : 1);    // super-tiles of the largest CTA
        *n_max_out = n_max;
        a.x_local = (!i8 && n_max < a.groups) ? 1 : 0;
        const int gstaged = a.x_local ? n_max : a.groups;
        size_t off = i8 ? (size_t)cols : (size_t)gstaged * nvt * 384;
        off = (off + 15) & ~(size_t)15;
        a.off_xcst = (int)off;
        off += i8 ? (size_t)a.groups * sizeof(int) : (size_t)gstaged * nvt * 16;
        off = (off + 15) & ~(size_t)15;
        a.off_part = (int)off;
        const int max_rb_per_cta = aligned ? (a.part_q + 1) : ((a.part_q + 1 + a.groups - 1) / a.groups + 1);
        off += (size_t)(max_rb_per_cta + kWarps) * kStRows * nvt * sizeof(float);
        if (fusedx) {
            off = (off + 15) & ~(size_t)15;
            a.off_xtmp = (int)off;
            off += (size_t)cols * sizeof(half) + 64 * sizeof(float);
        }
        off = (off + 15) & ~(size_t)15;
        a.off_bar = (int)off;
        off += (size_t)kMaxSlots * 8;
        a.off_gen = (int)off;
        off += (size_t)kMaxSlots * 4;
        off = (off + 127) & ~(size_t)127;
        a.off_ring = (int)off;
        return off;
    };

    // Whole row blocks per CTA -- no row block then spans two CTAs and nothing is combined across
    // CTAs -- in two cases: when that keeps the SMs at least 80 % evenly loaded; and when a CTA's
    // whole share of row blocks fits the ring that two co-resident CTAs allow, however few CTAs
    // that leaves: such a launch has all its weights on the chip before the kernel in front of
    // it ends, so its time after that is a few hundred nanoseconds of arithmetic either way,
    // while a combine across CTAs costs a store, a load and a poll on top.  Otherwise the
    // matrix is cut at super-tile granularity (K is split across CTAs).
    int grid = 0, n_max = 0;
    size_t off = layout(1, &grid, &n_max);
    bool aligned = force_aligned || (nrb >= grid_max && (double)nrb / ((double)per_cta_rb * grid_max) >= 0.8);
    if (!aligned && off + (size_t)n_max * kStBytes <= kCoResidentBytes && n_max <= kMaxSlots) aligned = true;
    if (!aligned) off = layout(0, &grid, &n_max);
    a.late_release = release_rule(rows, cols);
    // Ring: what a CTA can use, bounded by what lets two CTAs share the SM (the launch that
    // follows prefetches its weights beside this one); a problem whose activations leave less
    // than 24 slots that way runs one CTA per SM with all of the shared memory.
    const int want = n_max < kWarps ? kWarps : (n_max > kMaxSlots ? kMaxSlots : n_max);
    long long slots = ((long long)kCoResidentBytes - (long long)off) / kStBytes;
    if (slots < want && slots < 24) slots = ((long long)kMaxSmemBytes - (long long)off) / kStBytes;
    if (slots > want) slots = want;
    if (slots < kWarps)
        return fail(TLLM_ERR_SIZE, "rows=%d cols=%d with %d vectors per pass needs more shared memory than an SM has "
                    "(%zu bytes before the ring)", rows, cols, nvt, off);
    a.ring_slots = (int)slots;
    a.l2_prefetch = (n_max > (int)slots) ? 1 : 0;
    off += (size_t)slots * kStBytes;
    *grid_out = grid;
    *smem_out = off;
    return TLLM_OK;
}

template <int MODE, int NB, int NV, bool AR = false>
static int launch_mode(const GemvArgs& a, int grid, size_t smem, cudaStream_t stream)
{
    static bool attr[64] = {};
    static std::mutex mu;
    int dev = 0;
    cudaGetDevice(&dev);
    {
        std::lock_guard<std::mutex> lk(mu);
        if (dev >= 0 && dev < 64 && !attr[dev]) {
            const cudaError_t e1 = cudaFuncSetAttribute(gemv_packed_kernel<MODE, NB, NV, AR>,
                                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxSmemBytes);
            const cudaError_t e2 = cudaFuncSetAttribute(gemv_packed_kernel<MODE, NB, NV, AR>,
                                                        cudaFuncAttributePreferredSharedMemoryCarveout,
                                                        cudaSharedmemCarveoutMaxShared);
            if (e1 != cudaSuccess || e2 != cudaSuccess) {
                cudaGetLastError();
                return fail(TLLM_ERR_LAUNCH, "gemv_packed shared-memory set-up: %s",
                            cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
            }
            attr[dev] = true;
        }
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
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_packed_kernel<MODE, NB, NV, AR>, a);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(TLLM_ERR_LAUNCH, "gemv_packed launch: %s", cudaGetErrorString(e));
    }
    return TLLM_OK;
}

// Vectors per pass as instantiated for a batch of 1..4 FP16 vectors.
static inline int f16_nvt(int batch) { return batch <= 1 ? 1 : (batch == 2 ? 2 : 4); }

static int dispatch(const GemvArgs& a, int mode, int grid, size_t smem, cudaStream_t stream)
{
    switch (mode) {
        case kF16:
            if (a.batch <= 1) return launch_mode<kF16, 1, 1>(a, grid, smem, stream);
            if (a.batch == 2) return launch_mode<kF16, 1, 2>(a, grid, smem, stream);
            return launch_mode<kF16, 2, 2>(a, grid, smem, stream);
        case kI8Norm: return launch_mode<kI8Norm, 1, 1>(a, grid, smem, stream);
        case kI8Silu: return launch_mode<kI8Silu, 1, 1>(a, grid, smem, stream);
        case kI8Quant: return launch_mode<kI8Quant, 1, 1>(a, grid, smem, stream);
        default: return launch_mode<kI8, 1, 1>(a, grid, smem, stream);
    }
}

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

// x: half [batch, cols] (mode kF16, batch 1..4) or int8 [cols].
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
    a.batch = batch;
    int grid = 0;
    size_t smem = 0;
    if ((st = plan_gemv(a, s->sms, mode, mode == kF16 ? f16_nvt(batch) : 1, kMaxCtas, false, &grid, &smem))) return st;
    unsigned ticket;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        ticket = s->ticket++ % kTickets;
    }
    a.ws = s->ws + (size_t)ticket * kMaxCtas * 2 * kRecFloats;
    a.ws_stride = 2 * kRecFloats;
    a.err = s->misc + 1;
    return dispatch(a, mode, grid, smem, stream);
}

// Several matrices that share x and the column count (q/k/v; gate/up): matrices that were
// packed back to back (every row count but the last a multiple of 64) are one contiguous
// super-tile array and are streamed as ONE matrix in one launch, outputs scattered per
// segment; otherwise one launch each.
// x is FP16 (xq == nullptr) or INT8 with its scale in device memory.
static int gemv_packed_multi_any(int count, const uint8_t* const* packed, half* const* y, const int* rows, int cols,
                                 const half* x, const int8_t* xq, const float* scale_dev, cudaStream_t stream)
{
    const bool i8 = (xq != nullptr);
    if (count >= 2 && count <= TLLM_MAX_FUSED) {
        bool contiguous = true;
        SegY seg = {};
        seg.n = count;
        int total = 0;
        for (int i = 0; i < count; i++) {
            if (i + 1 < count)
                contiguous = contiguous && (rows[i] % kStRows == 0) && (packed[i + 1] == packed[i] + packed_bytes(rows[i], cols));
            seg.rows[i] = rows[i];
            seg.y[i] = y[i];
            total += rows[i];
        }
        if (contiguous)
            return i8 ? launch_packed_once(packed[0], xq, nullptr, 1.0f, kI8, 1, total, cols, stream, scale_dev, nullptr, &seg)
                      : launch_packed_once(packed[0], x, nullptr, 1.0f, kF16, 1, total, cols, stream, nullptr, nullptr, &seg);
    }
    for (int i = 0; i < count; i++) {
        const int st = i8 ? launch_packed_once(packed[i], xq, y[i], 1.0f, kI8, 1, rows[i], cols, stream, scale_dev)
                          : launch_gemv_packed(packed[i], x, y[i], 1, rows[i], cols, stream);
        if (st) return st;
    }
    return TLLM_OK;
}

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
    // up to four vectors share one pass over the weights; larger batches take ceil(B/4) passes.
    // Where the staged activations of that many vectors do not fit beside a ring in shared
    // memory (very long rows), fewer vectors share a pass.
    int per = kMaxVec;
    for (int b0 = 0; b0 < batch;) {
        const int nb = (batch - b0 >= per) ? per : (batch - b0);
        const int st = launch_packed_once(packed, x + (size_t)b0 * cols, y + (size_t)b0 * rows, 1.0f, kF16, nb, rows, cols,
                                          stream);
        if (st == TLLM_ERR_SIZE && per > 1) {
            per >>= 1;
            continue;
        }
        if (st) return st;
        b0 += nb;
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
// loads the library carries these 160 KB until the process exits.
//   [0, 163840)       partial-sum records, kNoAllocMaxCtas x 2 x 64 words {value, flag} (one vector)
//   [163840, 163844)  device error flag
constexpr int kNoAllocMaxRows = 65536;
constexpr int kNoAllocMaxCtas = 160;
constexpr size_t kNoAllocWsBytes = (size_t)kNoAllocMaxCtas * 2 * kStRows * sizeof(uint2);
constexpr size_t kNoAllocBytes = kNoAllocWsBytes + 256;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

struct NoAllocDevice {
    unsigned char* base = nullptr;   // device address of g_noalloc_scratch on this device
    int sms = 0;
};
static NoAllocDevice g_noalloc[64];

// Device address of the scratch array on the current device, looked up once per device under
// the library mutex (the address is stored last, so a reader that sees it sees the rest).
static int noalloc_device(NoAllocDevice** out)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(TLLM_ERR_DEVICE, "no usable current device");
    std::lock_guard<std::mutex> lk(g_mu);
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
    *out = &nd;
    return TLLM_OK;
}

// One FP16 vector, prepared weights, no allocation of any kind.  The first call on a
// device looks up the device address of the scratch array (cudaGetSymbolAddress, with
// that device current) and raises the kernel's shared-memory limit; make that first
// call outside any stream capture.  All calls share the one scratch array, which
// keeps what the previous call left: the records (their flags must start at zero) are
// cleared on `stream` before each launch, and two calls whose kernels overlap on the GPU
// (different streams) race.  With one vector a partial record is 64 words, so the records
// are laid out at that stride here (ws_stride), and the grid is capped at kNoAllocMaxCtas.
int launch_gemv_packed_noalloc(const uint8_t* packed, const half* x, half* y, int rows, int cols,
                               cudaStream_t stream)
{
    if (rows > kNoAllocMaxRows)
        return fail(TLLM_ERR_SIZE, "rows=%d exceeds the no-allocation variant's maximum of %d", rows, kNoAllocMaxRows);
    NoAllocDevice* nd = nullptr;
    int st = noalloc_device(&nd);
    if (st) return st;
    GemvArgs a = {};
    a.packed = packed;
    a.x = x;
    a.y = y;
    a.in_scale = 1.0f;
    a.rows = rows;
    a.cols = cols;
    a.batch = 1;
    int grid = 0;
    size_t smem = 0;
    if ((st = plan_gemv(a, nd->sms, kF16, 1, kNoAllocMaxCtas, false, &grid, &smem))) return st;
    a.ws = reinterpret_cast<uint2*>(nd->base);
    a.err = reinterpret_cast<int*>(nd->base + kNoAllocWsBytes);
    a.ws_stride = 2 * kStRows;
    // the records' flags must start at zero; a call that was cut short may have left some set
    if (cudaMemsetAsync(a.ws, 0, (size_t)grid * 2 * kStRows * sizeof(uint2), stream) != cudaSuccess) {
        cudaGetLastError();
        return fail(TLLM_ERR_LAUNCH, "clearing the scratch records failed");
    }
    return dispatch(a, kF16, grid, smem, stream);
}

// Synchronises `stream`, then reports and clears the error flag that the no-allocation
// entry point's kernels set when a bounded wait expires.  Allocates nothing.
int noalloc_error_check(cudaStream_t stream)
{
    NoAllocDevice* nd = nullptr;
    int st = noalloc_device(&nd);
    if (st) return st;
    int* flag_dev = reinterpret_cast<int*>(nd->base + kNoAllocWsBytes);
    int flag = 0;
    if (cudaMemcpyAsync(&flag, flag_dev, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess)
        return fail(TLLM_ERR_LAUNCH, "error flag read: %s", cudaGetErrorString(cudaGetLastError()));
    if (flag != 0) {
        cudaMemsetAsync(flag_dev, 0, sizeof(int), stream);
        return fail(flag, "a kernel reported status %d (bounded wait expired)", flag);
    }
    return TLLM_OK;
}

// Time-stamp buffer of the fused all-reduce per device (see GemvArgs::ar_trace); set by
// allreduce_set_trace, nullptr = off.
struct ArTrace { unsigned long long* buf = nullptr; int cap = 0; };
static ArTrace g_ar_trace[64];

int allreduce_set_trace(void* buffer, int records)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(TLLM_ERR_DEVICE, "no usable current device");
    if (buffer && records < 1) return fail(TLLM_ERR_SIZE, "trace buffer of %d records", records);
    std::lock_guard<std::mutex> lk(g_mu);
    g_ar_trace[dev].buf = static_cast<unsigned long long*>(buffer);
    g_ar_trace[dev].cap = buffer ? records : 0;
    return TLLM_OK;
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
    a.batch = 1;
    int grid = 0;
    size_t smem = 0;
    if ((st = plan_gemv(a, s->sms, kF16, 1, kMaxCtas, true, &grid, &smem))) return st;
    a.ws = s->ws;                       // unused in the aligned split
    a.err = s->misc + 1;
    a.ws_stride = 2 * kRecFloats;
    a.ar_world = world;
    a.ar_rank = rank;
    a.ar_rows_max = rows_max;
    for (int d = 0; d < world; d++) a.ar_recv[d] = static_cast<uint2*>(peer_recv[d]);
    a.ar_epoch = static_cast<unsigned*>(epoch_local);
    {
        int dev = 0;
        cudaGetDevice(&dev);
        std::lock_guard<std::mutex> lk(g_mu);
        if (dev >= 0 && dev < 64) {
            a.ar_trace = g_ar_trace[dev].buf;
            a.ar_trace_cap = g_ar_trace[dev].cap;
        }
    }
    return launch_mode<kF16, 1, 1, true>(a, grid, smem, stream);
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
    const long long threads = (long long)((rows + kStRows - 1) / kStRows) * (cols / kGroup) * 512;
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

int weight_unregister(const void* nz)
{
    std::lock_guard<std::mutex> lk(g_reg_mu);
    g_registry.erase(nz);
    return TLLM_OK;
}

}  // namespace tllm

#ifdef TLLM_TIMELINE
// host_out: [8][256][8] time stamps, counts: [256] launches seen per CTA index.
extern "C" int tllm_b200_timeline_read(unsigned long long* host_out, unsigned* counts)
{
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(host_out, tllm::g_tl, sizeof(tllm::g_tl)) != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(counts, tllm::g_tl_cnt, sizeof(tllm::g_tl_cnt)) != cudaSuccess) return -1;
    return 0;
}
#endif
