// Ternary GEMV on the 5th-generation tensor cores (tcgen05, INT8), one activation vector.
//
// Same arithmetic as gemv_mma.cu -- weights expanded to INT8 {-1,0,+1} with PRMT, FP16
// activations as three unsigned byte digits of a per-group block fixed point plus a row of
// ones, exact INT32 group sums, one FP32 multiply by scale * 2^(e-22) per group -- but the
// contraction runs as tcgen05.mma.kind::i8 with the weights in TENSOR MEMORY:
//
//   unit      128 weight rows (a "strip" of 8 row blocks) x one scale group of 128 columns.
//   expanders 16 warps = 4 quads of 128 threads.  A thread owns one row of the strip (its
//             TMEM lane): it reads the row's 32 bytes of pair codes from the warp's ring in
//             shared memory, expands them with 32 PRMTs and writes them with tcgen05.st as
//             two half-units of 16 columns.  Nothing of the expansion is replicated across
//             lanes, and the epilogue below runs once per row instead of once per MMA
//             fragment lane, which is what made the mma.sync formulation issue-bound.
//   issuer    one thread of a 17th warp issues, for every half-unit, two tcgen05.mma
//             (M = 128, N = 16, K = 32): A from tensor memory, B = the activation digits in
//             shared memory (128-byte-swizzled rows d0, d1, d2, ones), D = a 128 x 16 INT32
//             accumulator per unit in tensor memory; tcgen05.commit releases the slots.
//   epilogue  the row's thread reads its accumulator (tcgen05.ld, 4 columns), combines the
//             digits, converts once and adds scale * 2^(e-22) * sum to its FP32 accumulator.
//
// Work split: units are numbered strip-major and dealt to the CTAs (one per SM) in
// contiguous, equal ranges, then to the 4 quads of a CTA in contiguous runs, so a warp's
// tiles of consecutive units are contiguous in memory (two tiles of one row block per
// bulk copy).  A strip that spans several CTAs is combined by the CTA that arrives last,
// in CTA order, as in gemv_mma.cu.  Tensor memory: 256 columns per CTA (two CTAs per SM):
// per quad two 16-column weight slots and two 16-column accumulators.
//
// Every wait is bounded; a wait that gives up raises an abort flag that all roles poll,
// the device error flag is set, and the kernel falls through to the exit that frees TMEM.
#include <mutex>

#include "launch.cuh"
#include "packed_layout.cuh"

namespace tllm {

namespace tc5 {

constexpr int kQuads = 4;
constexpr int kExpThreads = kQuads * 128;
constexpr int kThreads = kExpThreads + 32;        // + the issuer warp
constexpr int kStripRows = 128;
constexpr int kStripBlocks = kStripRows / kTileRows;   // 8 row blocks
constexpr int kSlotUnits = 2;                     // units per ring slot
constexpr int kRing = 2;                          // ring slots per warp
constexpr int kSlotBytes = kSlotUnits * 2 * kTileBytes;     // two row blocks x two units
constexpr int kTmemCols = 256;
constexpr int kQuadCols = 64;                     // per quad: A0 A1 (16 each) D0 D1 (16 each)
constexpr int kMaxCtas = 256;
constexpr int kTickets = 16;
constexpr int kMaxStrips = 1 << 13;

struct Args {
    const uint8_t* packed;
    const void* x;            // half [cols] or int8 [cols]
    half* y;
    float in_scale;
    const float* in_scale_dev;
    int rows, cols, groups, nrb, nstrips;
    int int8;                 // 1: INT8 activations
    int part_q, part_r;       // units = grid * part_q + part_r
    float* ws;                // [grid][2][128] partial records of this ticket
    int* counters;            // [nstrips]
    int* err;
    int off_xfac, off_part, off_ring, off_bar;    // shared memory carve-up (digits start at 0)
    int nseg;                 // outputs of matrices packed back to back (see gemv_mma.cu)
    int seg_row[TLLM_MAX_FUSED + 1];
    half* seg_y[TLLM_MAX_FUSED];
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// Bounded wait; false = gave up (also when another role already reported an error).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag)
{
#pragma unroll 1
    for (int i = 0; i < (1 << 22); i++) {
        if (mbar_try(bar, parity)) return true;
        if ((i & 1023) == 1023 && *abort_flag) return false;
    }
    return false;
}
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
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, int (&r)[4])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
}
// Shared-memory descriptor of the activation operand: K-major rows of 128 bytes with the
// 128-byte swizzle, one 8-row atom of 1024 bytes per scale group.  The instruction's N is 16;
// the stride between 8-row atoms is 0, so rows 8..15 re-read rows 0..7 (their accumulator
// columns are never looked at) and a group costs 1 KB of shared memory instead of 2.
__device__ __forceinline__ uint64_t make_b_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;                                 // leading byte offset (unused with swizzle)
    d |= (uint64_t)0 << 32;                                 // stride byte offset between 8-row atoms
    d |= (uint64_t)1 << 46;                                 // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                                 // layout: 128-byte swizzle
    return d;
}
// kind::i8 instruction descriptor: S8 weights x (U8 digits | S8 activations) -> S32, K-major.
__device__ __forceinline__ uint32_t make_idesc(bool b_signed)
{
    uint32_t d = 0;
    d |= 2u << 4;                          // D format S32
    d |= 1u << 7;                          // A format S8
    d |= (b_signed ? 1u : 0u) << 10;       // B format
    d |= (uint32_t)(16 >> 3) << 17;        // N = 16
    d |= (uint32_t)(128 >> 4) << 24;       // M = 128
    return d;
}
__device__ __forceinline__ void mma_ts_i8(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p; }"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ int part_start(int c, int q, int r) { return c * q + min(c, r); }
__device__ __forceinline__ int part_of(int u, int q, int r)
{
    const int big = r * (q + 1);
    return (u < big) ? (int)((unsigned)u / (unsigned)(q + 1)) : r + (int)((unsigned)(u - big) / (unsigned)q);
}
__device__ __forceinline__ int run_start(int quad, int n) { return (quad * n) >> 2; }

__device__ __forceinline__ half* out_ptr(const Args& a, int r)
{
    if (a.nseg == 0) return a.y + r;
    int i = 0;
#pragma unroll
    for (int k = 1; k < TLLM_MAX_FUSED; k++)
        if (k < a.nseg && r >= a.seg_row[k]) i = k;
    return a.seg_y[i] + (r - a.seg_row[i]);
}

// Byte offset of activation byte k (0..127) of digit row j (0..7) inside a group's 1 KB atom.
__device__ __forceinline__ int b_off(int j, int k) { return j * 128 + ((((k >> 4) ^ j) & 7) << 4) + (k & 15); }

// FP16 activations -> digit rows of every group (block fixed point, see gemv_mma.cu).  Each
// thread converts 8 consecutive activations; 16 threads cover a group.
__device__ __forceinline__ void stage_digits(const half* __restrict__ x, int cols, uint8_t* xdig, float* xfac, int tid)
{
    const int items = cols >> 3;
    for (int base = 0; base < items; base += kExpThreads) {
        const int item = base + tid;
        const bool valid = item < items;                    // uniform per half-warp (items % 16 == 0)
        const int ic = valid ? item : 0;
        const int g = ic >> 4, l16 = ic & 15;
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x) + ic);
        const half* h = reinterpret_cast<const half*>(&raw);
        float f[8];
        float m = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            f[j] = __half2float(h[j]);
            m = fmaxf(m, fabsf(f[j]));
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const int e = max((int)((__float_as_uint(m) >> 23) & 0xffu) - 126, -24);
        const float up = (m > 0.f) ? __uint_as_float((uint32_t)(22 - e + 127) << 23) : 0.f;
        const float dn = (m > 0.f) ? __uint_as_float((uint32_t)(e - 22 + 127) << 23) : 0.f;
        uint32_t d[3][2] = {{0, 0}, {0, 0}, {0, 0}};
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t q = (uint32_t)(__float2int_rn(f[j] * up) + (1 << 23));
            d[0][j >> 2] |= (q & 0xffu) << (8 * (j & 3));
            d[1][j >> 2] |= ((q >> 8) & 0xffu) << (8 * (j & 3));
            d[2][j >> 2] |= ((q >> 16) & 0xffu) << (8 * (j & 3));
        }
        if (valid) {
            uint8_t* atom = xdig + (size_t)g * 1024;
            const int k = l16 * 8;
#pragma unroll
            for (int j = 0; j < 3; j++) *reinterpret_cast<uint2*>(atom + b_off(j, k)) = make_uint2(d[j][0], d[j][1]);
            *reinterpret_cast<uint2*>(atom + b_off(3, k)) = make_uint2(0x01010101u, 0x01010101u);
#pragma unroll
            for (int j = 4; j < 8; j++) *reinterpret_cast<uint2*>(atom + b_off(j, k)) = make_uint2(0u, 0u);
            if (l16 == 0) xfac[g] = dn;
        }
    }
}

// INT8 activations: row 0 carries the vector, rows 1..7 are zero.
__device__ __forceinline__ void stage_int8(const int8_t* __restrict__ x, int cols, uint8_t* xdig, int tid)
{
    const int items = cols >> 3;
    for (int item = tid; item < items; item += kExpThreads) {
        const int g = item >> 4, k = (item & 15) * 8;
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(x) + item);
        uint8_t* atom = xdig + (size_t)g * 1024;
        *reinterpret_cast<uint2*>(atom + b_off(0, k)) = v;
#pragma unroll
        for (int j = 1; j < 8; j++) *reinterpret_cast<uint2*>(atom + b_off(j, k)) = make_uint2(0u, 0u);
    }
}

__global__ void __launch_bounds__(kThreads, 2) gemv_tc5_kernel(const Args a)
{
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the 128-byte swizzle atoms of the activation operand
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bars[kQuads * 8];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    asm volatile("griddepcontrol.launch_dependents;");
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.groups;
    const int u_lo = part_start(blockIdx.x, a.part_q, a.part_r);
    const int n = a.part_q + ((int)blockIdx.x < a.part_r ? 1 : 0);       // units of this CTA
    const int strip_first = (int)((unsigned)u_lo / (unsigned)G);
    const int strip_last = (int)((unsigned)(u_lo + n - 1) / (unsigned)G);

    uint8_t* xdig = smem;                                              // [G][1024]
    float* xfac = reinterpret_cast<float*>(smem + a.off_xfac);          // [G]
    float* part = reinterpret_cast<float*>(smem + a.off_part);          // [local strips][quad][128]
    const uint32_t bar0 = smem_u32(bars);
    auto full_a = [&](int q, int s) { return bar0 + 8u * (q * 8 + s); };
    auto empty_a = [&](int q, int s) { return bar0 + 8u * (q * 8 + 2 + s); };
    auto d_full = [&](int q, int s) { return bar0 + 8u * (q * 8 + 4 + s); };
    auto d_empty = [&](int q, int s) { return bar0 + 8u * (q * 8 + 6 + s); };

    if (tid == 0) {
        for (int q = 0; q < kQuads; q++)
            for (int s = 0; s < 2; s++) {
                mbar_init(full_a(q, s), 128);
                mbar_init(empty_a(q, s), 1);
                mbar_init(d_full(q, s), 1);
                mbar_init(d_empty(q, s), 128);
            }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == kQuads * 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // partial sums start at zero (a quad that never touches a strip leaves its slot alone)
    {
        const int nloc = strip_last - strip_first + 1;
        for (int i = tid; i < nloc * kQuads * kStripRows; i += kThreads) part[i] = 0.f;
    }

    // ---- this warp's ring and its first fetches (weights are constants: before the wait) ----
    const int quad = warp >> 2, wq = warp & 3;                          // expander warps only
    const int r_lo = u_lo + run_start(quad < kQuads ? quad : 0, n);
    const int r_hi = u_lo + run_start((quad < kQuads ? quad : 0) + 1, n);
    const uint32_t ring = smem_u32(smem + a.off_ring) + warp * (kRing * kSlotBytes);
    const uint8_t* ring_p = smem + a.off_ring + warp * (kRing * kSlotBytes);
    const uint32_t rbar = smem_u32(smem + a.off_bar) + warp * (kRing * 8);
    if (warp < kQuads * 4 && lane == 0) {
        for (int s = 0; s < kRing; s++) mbar_init(rbar + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    // Chunk c of a run: up to kSlotUnits units that lie in one strip.  fetch() is called by
    // lane 0 with the first unit of the chunk and returns the number of units it covers.
    auto chunk_len = [&](int u) {
        const int g = u - (int)((unsigned)u / (unsigned)G) * G;
        return min(kSlotUnits, min(G - g, r_hi - u));
    };
    auto fetch = [&](int u, int slot) {
        const int strip = (int)((unsigned)u / (unsigned)G), g = u - strip * G;
        const int nu = chunk_len(u);
        const int rb0 = strip * kStripBlocks + wq * 2;                   // this warp's two row blocks
        uint32_t bytes = 0;
        for (int j = 0; j < 2; j++)
            if (rb0 + j < a.nrb) bytes += (uint32_t)nu * kTileBytes;
        if (bytes == 0) return;
        mbar_expect_tx(rbar + slot * 8, bytes);
        for (int j = 0; j < 2; j++)
            if (rb0 + j < a.nrb)
                bulk_g2s(ring + slot * kSlotBytes + j * (kSlotUnits * kTileBytes),
                         a.packed + ((size_t)(rb0 + j) * G + g) * kTileBytes, (uint32_t)nu * kTileBytes, rbar + slot * 8);
    };
    int fetch_u = r_lo;            // next unit to request (lane 0 of expander warps)
    int fetch_c = 0;
    if (warp < kQuads * 4 && lane == 0) {
        for (int s = 0; s < kRing && fetch_u < r_hi; s++) {
            fetch(fetch_u, fetch_c % kRing);
            fetch_u += chunk_len(fetch_u);
            fetch_c++;
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_slot;
    volatile int* abortp = &abort_flag;

    // ---- everything below may depend on the previous kernel in the stream -------------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid < kExpThreads) {
        if (a.int8) stage_int8(reinterpret_cast<const int8_t*>(a.x), a.cols, xdig, tid);
        else stage_digits(reinterpret_cast<const half*>(a.x), a.cols, xdig, xfac, tid);
    }
    // the digits were written with ordinary stores and are read by the tensor core
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();

    if (warp == kQuads * 4) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc(a.int8 != 0);
            const uint32_t xb = smem_u32(xdig);
            int nu_q[kQuads], u_q[kQuads];
            int rounds = 0;
            for (int q = 0; q < kQuads; q++) {
                u_q[q] = u_lo + run_start(q, n);
                nu_q[q] = run_start(q + 1, n) - run_start(q, n);
                rounds = max(rounds, 2 * nu_q[q]);
            }
            bool ok = true;
            for (int hu = 0; hu < rounds && ok; hu++) {
                const int h = hu & 1, i = hu >> 1, dslot = i & 1;
                for (int q = 0; q < kQuads && ok; q++) {
                    if (i >= nu_q[q]) continue;
                    const int u = u_q[q] + i;
                    const int g = u - (int)((unsigned)u / (unsigned)G) * G;
                    ok = mbar_wait(full_a(q, h), (uint32_t)i & 1u, abortp);
                    if (ok && h == 0) ok = mbar_wait(d_empty(q, dslot), ((uint32_t)(i >> 1) & 1u) ^ 1u, abortp);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_t = tmem + q * kQuadCols + h * 16;
                    const uint32_t d_t = tmem + q * kQuadCols + 32 + dslot * 16;
#pragma unroll
                    for (int kk = 0; kk < 2; kk++) {
                        const uint64_t bd = make_b_desc(xb + g * 1024 + (2 * h + kk) * 32);
                        mma_ts_i8(d_t, a_t + kk * 8, bd, idesc, (h > 0 || kk > 0) ? 1u : 0u);
                    }
                    mma_commit(empty_a(q, h));
                    if (h == 1) mma_commit(d_full(q, dslot));
                }
            }
            if (!ok) abort_flag = 1;
        }
    } else {
        // ---------------- expanders / epilogue: one thread per row of the strip ----------------
        const int row = wq * 32 + lane;                                  // row inside the strip = TMEM lane
        const uint32_t lane_base = tmem + ((uint32_t)(wq * 32) << 16) + quad * kQuadCols;
        const int jblk = lane >> 4, r16 = lane & 15;                      // row block (of the warp's two) and row in it
        const int spos = (r16 < 8) ? 2 * r16 : 2 * (r16 - 8) + 1;
        const int nu = r_hi - r_lo;
        float acc = 0.f;
        int acc_strip = -1;
        bool ok = true;
        float sc_prev = 0.f;
        int g_prev = 0, strip_prev = 0;

        auto flush = [&]() {
            if (acc_strip >= 0) part[((acc_strip - strip_first) * kQuads + quad) * kStripRows + row] = acc;
            acc = 0.f;
        };
        auto epilogue = [&](int i_prev) -> bool {                         // accumulator of unit i_prev
            const int dslot = i_prev & 1;
            if (!mbar_wait(d_full(quad, dslot), (uint32_t)(i_prev >> 1) & 1u, abortp)) return false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            int d[4];
            tmem_ld4(lane_base + 32 + dslot * 16, d);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(d_empty(quad, dslot));
            if (strip_prev != acc_strip) {
                flush();
                acc_strip = strip_prev;
            }
            if (a.int8) {
                acc = fmaf((float)d[0], sc_prev, acc);
            } else {
                const int p = d[0] + d[1] * 256 + (d[2] - 128 * d[3]) * 65536;     // |p| <= 2^30
                acc = fmaf((float)p, sc_prev * xfac[g_prev], acc);
            }
            return true;
        };

        int u = r_lo, chunk_c = 0, in_chunk = 0, chunk_n = 0;
        for (int i = 0; i < nu && ok; i++, u++) {
            const int strip = (int)((unsigned)u / (unsigned)G), g = u - strip * G;
            if (in_chunk == chunk_n) {                                    // next ring slot
                if (i > 0) chunk_c++;
                chunk_n = chunk_len(u);
                in_chunk = 0;
                const int rb0 = strip * kStripBlocks + wq * 2;
                if (rb0 < a.nrb)                                          // uniform per warp: something was requested
                    ok = mbar_wait(rbar + (chunk_c % kRing) * 8, (uint32_t)(chunk_c / kRing) & 1u, abortp);
                if (!ok) break;
            }
            const int rb = strip * kStripBlocks + wq * 2 + jblk;
            const uint8_t* tp = ring_p + (chunk_c % kRing) * kSlotBytes + jblk * (kSlotUnits * kTileBytes) + in_chunk * kTileBytes;
            uint4 c0, c1;
            float sc = 0.f;
            if (rb < a.nrb) {
                c0 = *reinterpret_cast<const uint4*>(tp + r16 * 32);
                c1 = *reinterpret_cast<const uint4*>(tp + r16 * 32 + 16);
                sc = __half2float(*(reinterpret_cast<const half*>(tp + kTileCodeBytes) + spos));
            } else {                                                      // rows past the matrix: the (0,0) pair code
                c0 = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
                c1 = c0;
            }
            in_chunk++;
            if (in_chunk == chunk_n) {                                    // slot consumed: request the chunk two ahead
                __syncwarp();
                if (lane == 0 && fetch_u < r_hi) {
                    fetch(fetch_u, fetch_c % kRing);
                    fetch_u += chunk_len(fetch_u);
                    fetch_c++;
                }
            }
            const uint32_t w[4][2] = {{c0.x, c0.y}, {c0.z, c0.w}, {c1.x, c1.y}, {c1.z, c1.w}};
#pragma unroll
            for (int h = 0; h < 2; h++) {
                if (!mbar_wait(empty_a(quad, h), ((uint32_t)i & 1u) ^ 1u, abortp)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t r[16];
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    const uint32_t lo = w[t][h], hi = lo >> 16;
                    r[t] = prmt(kTabA_lo, kTabA_hi, lo);                  // K 64h + 4t..      (column t)
                    r[4 + t] = prmt(kTabB_lo, kTabB_hi, lo);              // K 64h + 16 + 4t.. (column 4 + t)
                    r[8 + t] = prmt(kTabA_lo, kTabA_hi, hi);              // K 64h + 32 + 4t..
                    r[12 + t] = prmt(kTabB_lo, kTabB_hi, hi);             // K 64h + 48 + 4t..
                }
                tmem_st16(lane_base + h * 16, r);
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(full_a(quad, h));
            }
            if (!ok) break;
            if (i > 0) ok = epilogue(i - 1);
            sc_prev = sc;
            g_prev = g;
            strip_prev = strip;
        }
        if (ok && nu > 0) ok = epilogue(nu - 1);
        flush();
        if (!ok) abort_flag = 1;
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (abort_flag) {
        if (tid == 0) atomicExch(a.err, TLLM_ERR_TIMEOUT);
    } else {
        // ---- reduction: quads of this CTA, then CTAs, strip by strip -----------------------------
        const float oscale = a.int8 ? (a.in_scale_dev ? __ldg(a.in_scale_dev) : a.in_scale) : 1.0f;
        float* myrec = a.ws + (size_t)blockIdx.x * 2 * kStripRows;
        __shared__ int s_last;
        for (int s = strip_first; s <= strip_last; s++) {
            const int ua = max(u_lo, s * G), ub = min(u_lo + n, (s + 1) * G);
            const bool full = (ub - ua == G);
            float v = 0.f;
            int r = 0;
            if (tid < kStripRows) {
                const float* p = part + (size_t)(s - strip_first) * kQuads * kStripRows + tid;
                v = (p[0] + p[kStripRows]) + (p[2 * kStripRows] + p[3 * kStripRows]);
                r = s * kStripRows + tid;
                if (full) {
                    if (r < a.rows) *out_ptr(a, r) = __float2half_rn(v * oscale);
                } else {
                    myrec[((s == strip_first) ? 0 : 1) * kStripRows + tid] = v;
                    __threadfence();
                }
            }
            if (full) continue;
            __syncthreads();
            int c_a = 0, c_b = 0;
            if (tid == 0) {
                c_a = part_of(s * G, a.part_q, a.part_r);
                c_b = part_of((s + 1) * G - 1, a.part_q, a.part_r);
                const int prev = atomicAdd(a.counters + s, 1);
                s_last = (prev == c_b - c_a) ? 1 : 0;
                if (s_last) a.counters[s] = 0;
            }
            __syncthreads();
            if (s_last && tid < kStripRows) {
                __threadfence();
                c_a = part_of(s * G, a.part_q, a.part_r);
                c_b = part_of((s + 1) * G - 1, a.part_q, a.part_r);
                float tot = 0.f;
                for (int c = c_a; c <= c_b; c++) {
                    const int c_first = (int)((unsigned)part_start(c, a.part_q, a.part_r) / (unsigned)G);
                    tot += __ldcg(a.ws + (size_t)c * 2 * kStripRows + ((s == c_first) ? 0 : kStripRows) + tid);
                }
                if (r < a.rows) *out_ptr(a, r) = __float2half_rn(tot * oscale);
            }
            __syncthreads();
        }
    }
    __syncthreads();
    if (warp == kQuads * 4) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

struct Scratch {
    float* ws = nullptr;
    int* counters = nullptr;
    int sms = 0;
    unsigned ticket = 0;
    bool ready = false;
};
static Scratch g_scratch[64];
static std::mutex g_mu;

static int get_scratch(Scratch** out)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(TLLM_ERR_DEVICE, "no current CUDA device");
    std::lock_guard<std::mutex> lk(g_mu);
    Scratch& s = g_scratch[dev];
    if (!s.ready) {
        cudaDeviceGetAttribute(&s.sms, cudaDevAttrMultiProcessorCount, dev);
        const size_t wsb = (size_t)kTickets * kMaxCtas * 2 * kStripRows * sizeof(float);
        const size_t cb = (size_t)kTickets * kMaxStrips * sizeof(int);
        if (cudaMalloc(&s.ws, wsb) != cudaSuccess || cudaMalloc(&s.counters, cb) != cudaSuccess) {
            cudaGetLastError();
            return fail(TLLM_ERR_LAUNCH, "gemv_tc5: scratch allocation failed");
        }
        cudaMemset(s.counters, 0, cb);
        cudaFuncSetAttribute(gemv_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(gemv_tc5_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        s.ready = true;
    }
    *out = &s;
    return TLLM_OK;
}

}  // namespace tc5

bool gemv_tc5_supported(int rows, int cols)
{
    const int nstrips = (rows + tc5::kStripRows - 1) / tc5::kStripRows;
    return cols % kGroup == 0 && cols >= kGroup && nstrips <= tc5::kMaxStrips && (size_t)(cols / kGroup) * 1024 <= 64 * 1024;
}

// One activation vector (FP16, or INT8 with its scale by value or in device memory) against a
// prepared matrix; seg_* as in gemv_mma.cu (nseg == 0: y).  TLLM_ERR_SIZE: not supported.
int launch_gemv_tc5(const uint8_t* packed, const half* x, const int8_t* xq, float in_scale, const float* in_scale_dev,
                    half* y, int rows, int cols, int nseg, const int* seg_rows, half* const* seg_y, cudaStream_t stream)
{
    using namespace tc5;
    if (!gemv_tc5_supported(rows, cols)) return TLLM_ERR_SIZE;
    Scratch* s = nullptr;
    int st = get_scratch(&s);
    if (st) return st;
    Args a = {};
    a.packed = packed;
    a.x = xq ? (const void*)xq : (const void*)x;
    a.int8 = xq ? 1 : 0;
    a.y = y;
    a.in_scale = in_scale;
    a.in_scale_dev = in_scale_dev;
    a.rows = rows;
    a.cols = cols;
    a.groups = cols / kGroup;
    a.nrb = (rows + kTileRows - 1) / kTileRows;
    a.nstrips = (rows + kStripRows - 1) / kStripRows;
    a.nseg = nseg;
    int r0 = 0;
    for (int i = 0; i < nseg; i++) {
        a.seg_row[i] = r0;
        a.seg_y[i] = seg_y[i];
        r0 += seg_rows[i];
    }
    for (int i = nseg; i <= TLLM_MAX_FUSED; i++) a.seg_row[i] = r0;
    const int units = a.nstrips * a.groups;
    int grid = s->sms < kMaxCtas ? s->sms : kMaxCtas;
    if (units < grid) grid = units;
    a.part_q = units / grid;
    a.part_r = units % grid;
    unsigned ticket;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        ticket = s->ticket++ % kTickets;
    }
    a.ws = s->ws + (size_t)ticket * kMaxCtas * 2 * kStripRows;
    a.counters = s->counters + (size_t)ticket * kMaxStrips;
    a.err = device_error_flag();
    size_t off = (size_t)a.groups * 1024;
    a.off_xfac = (int)off;
    off += (size_t)a.groups * sizeof(float);
    off = (off + 15) & ~(size_t)15;
    a.off_part = (int)off;
    const int max_strips = (a.part_q + 1 + a.groups - 1) / a.groups + 1;
    off += (size_t)max_strips * kQuads * kStripRows * sizeof(float);
    off = (off + 15) & ~(size_t)15;
    a.off_ring = (int)off;
    off += (size_t)kQuads * 4 * kRing * kSlotBytes;
    a.off_bar = (int)off;
    off += (size_t)kQuads * 4 * kRing * 8;
    off += 1024;                                       // alignment slack
    if (off > 200 * 1024) return TLLM_ERR_SIZE;
    return launch_pdl("gemv_tc5", gemv_tc5_kernel, dim3(grid), dim3(kThreads), off, stream, a);
}

}  // namespace tllm
