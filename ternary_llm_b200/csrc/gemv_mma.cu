// Streaming ternary GEMV on the packed layout (packed_layout.cuh), sm_100a.
//
// The GEMV is HBM-bound: 2.125 bits per weight must stream at several TB/s, which
// leaves about 1.5 issue slots per weight per lane.  A masked add per weight on the
// CUDA cores costs 3-5, so the +x/-x/0 selection runs on the tensor cores instead.
// Weights are stored as 2-bit offset codes c = t + 1, sixteen to a word, arranged so
// that ONE logic instruction, `word & (0x03030303 << 2f)`, is an A-operand register of
// mma.sync.m16n8k32 (unsigned bytes c * 4^f of the 32 columns 32f..32f+31 of a 16-row x
// 128-column tile).  The B operand carries the activations as small signed digits, and the
// digits of the even steps (f = 0, 2) are stored multiplied by 4: then steps 0 and 1 both
// carry the factor 4 and accumulate in one MMA chain, steps 2 and 3 both carry 64 and
// accumulate in a second, and D_lo * 16 + D_hi = 64 * sum(c*x) exactly, in integers.
// sum(t*x) = sum(c*x) - sum(x) with sum(x) made once per group when the activations are
// staged; the factor 64 is divided out in FP32 with the scale.
//
//   FP16 activations: each scale group of 128 activations is converted once per CTA to
//   block fixed point, q = rint(x * 2^(22-e)) with 2^e > max|x| of the group, stored as
//   four BALANCED base-64 digits, q = d0 + 64 d1 + 4096 d2 + 262144 d3 with d in [-32,31]
//   (the 6-bit fields of q + 32*(1+64+64^2+64^3), each minus 32), so that a digit times 4
//   still is a signed byte.  A vector occupies four B columns; two vectors share one MMA,
//   up to four take two MMAs per operand register.  Every digit sum is exact in INT32 and
//   is converted to FP32 once per group and row.  Rounding x to 23 bits below the group
//   maximum is at the level of FP32 accumulation rounding itself.  A group that holds a
//   NaN or an infinity makes its outputs NaN, as FP32 accumulation of x would.
//   INT8 activations (ternary_gemv_int8 semantics): the vector as two digit columns,
//   x = lo + 16 hi with lo = x & 15 and hi = x >> 4; integer group sums stay exact.
//
// Work decomposition: the matrix is a linear array of tiles (16 rows x one scale group,
// 544 bytes; row-block major).  They are dealt to CTAs (one per SM) and, inside a CTA, to
// 16 warps in contiguous, equal ranges: whole 16-row blocks per CTA where that balances
// the SMs (or where a CTA's share fits its ring anyway), otherwise K is split across
// CTAs.  A warp walks its range in chunks of four tiles.  Weights arrive through a ring
// of R slots per CTA (a chunk per slot; 16-byte cp.async copies issued by all lanes of a
// warp, completion counted on one mbarrier per slot -- measured on this part, a ring fed
// by cp.async.bulk tops out near 4 TB/s over the whole GPU whatever its depth, while
// per-thread loads reach the full HBM rate).  R is what the shared-memory budget allows
// (two CTAs per SM: one computing, the next launch prefetching); the slots are dealt to
// the warps as private rings of depth R/16, the first R mod 16 warps one deeper, so every
// slot is filled and emptied by one warp in program order (no cross-warp hand-over, no
// parity wait on a barrier that is a phase behind) and a refill is one pointer increment.
// The first `depth` chunks of every warp are requested at kernel start.  Partial sums of a
// 16-row block are combined in a fixed order: first over the warps of a CTA, then, for a
// block that spans several CTAs, by the LAST of those CTAs: the others store their sums
// as 8-byte {value, flag} words (one store each, no fence, no atomic) and leave; the
// last one polls -- bounded -- for the flags, adds the records in CTA order, writes the
// outputs and clears the words for the next launch.  Results therefore do not depend on
// timing.  (An arrival counter with fences on both sides costs four dependent round
// trips to L2 per launch, about 3 us on this part; this costs one store and one load.)
//
// Launches carry the programmatic-dependent-launch attribute: the weight fetch is
// issued before griddepcontrol.wait (weights are constants), activations are read
// and outputs written after it, so a GEMV's weight stream starts while the kernel
// before it in the stream drains.  Every wait is bounded; a wait that gives up records
// TLLM_ERR_TIMEOUT in a device flag and the kernel returns.
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "packed_layout.cuh"
#include "launch.cuh"

namespace tllm {

constexpr int kWarpsLog2 = 4;
constexpr int kWarps = 1 << kWarpsLog2;
constexpr int kThreads = kWarps * 32;
constexpr int kTickets = 16;                          // independent scratch regions
constexpr int kMaxCtas = 256;
constexpr int kMaxVec = 4;                            // vectors per weight pass
#ifndef TLLM_GEMV_SLOT_TILES
#define TLLM_GEMV_SLOT_TILES 4
#endif
constexpr int kSlotTiles = TLLM_GEMV_SLOT_TILES;      // tiles per chunk = per ring slot
constexpr int kSlotBytes = kSlotTiles * kTileBytes;   // 2176
constexpr int kMaxSlots = 400 / kSlotTiles;           // ring slots per CTA, upper bound
constexpr int kRecFloats = kTileRows * kMaxVec;       // one partial record: 16 rows x 4 vectors
constexpr int kMaxPeers = TLLM_MAX_PEERS;
// Dynamic shared memory of one CTA when two are to share an SM (228 KB per SM, 1 KB
// reserved per resident CTA).
#ifndef TLLM_GEMV_CORESIDENT_BYTES
#define TLLM_GEMV_CORESIDENT_BYTES (112 * 1024)
#endif
constexpr size_t kCoResidentBytes = TLLM_GEMV_CORESIDENT_BYTES;
// A ring that two co-resident CTAs allow but that holds fewer slots than this (and less than the
// CTA's whole share) is given up for one CTA per SM with all of the shared memory.  Measured,
// the step from co-resident to alone costs far more than a shallow ring does (the launches either
// side lose their overlap: 8B sweep 0.87 -> 1.02 ms with the limit at 32; the 8192 x 28672 launch
// of the 70B stack 17 -> 38 us when its ring fell from 24 to 23 slots with the limit at 24), so
// the limit is the minimum of one slot per warp.
#ifndef TLLM_GEMV_PAIR_STAGING
#define TLLM_GEMV_PAIR_STAGING 1
#endif
#ifndef TLLM_GEMV_KSPLIT
#define TLLM_GEMV_KSPLIT 1
#endif
#ifndef TLLM_GEMV_KSPLIT_MIN_COLS
#define TLLM_GEMV_KSPLIT_MIN_COLS 12288
#endif
#ifndef TLLM_GEMV_MIN_SHARED_SLOTS
#define TLLM_GEMV_MIN_SHARED_SLOTS 16
#endif
constexpr int kMinSharedSlots = TLLM_GEMV_MIN_SHARED_SLOTS;
constexpr size_t kMaxSmemBytes = 226 * 1024;      // dynamic part; the kernel also has a few static bytes
// How far beyond the ring a warp asks for its weights to be brought into L2, in chunks (0 = off).
// The ring is bounded by shared memory: 63 KB in flight per SM at the 2 us an HBM access takes
// under load is 33 GB/s per SM, three quarters of the HBM rate.  The 126 MB L2 is the buffer that
// decouples the HBM stream from the chain of dependent launches: with this set, each warp prefetches (one
// prefetch.global.L2 per 128-byte line, no shared memory, no registers) the chunks it will copy
// into the ring a few iterations later, starting in the prologue -- that is, while the kernel
// in front of this one still runs -- so the ring's copies hit L2.  (cp.async.bulk.prefetch.L2 was
// measured first and did not help: like the bulk copy itself it is bound by its own engine.)
#ifndef TLLM_GEMV_L2_AHEAD_CHUNKS
#define TLLM_GEMV_L2_AHEAD_CHUNKS 0
#endif
constexpr int kL2Ahead = TLLM_GEMV_L2_AHEAD_CHUNKS;

// kI8Norm / kI8Silu / kI8Quant: INT8 arithmetic like kI8, but the activation vector is
// produced inside the kernel's staging phase from FP16 inputs (stage_x_fused below).
// kF16W: FP16 activations, four vectors per MMA column block on 16-bit block fixed point (two
// 8-bit digits per vector) instead of two vectors on 24 bits: batches of three and more.
// kF16Norm: FP16 arithmetic like kF16 (one vector), the vector is rmsnorm(fx_a (+ fx_b)) * fx_w made in
// the staging phase (the FP16-rounded sum goes to fx_res_out), as kI8Norm does for the INT8 path.
enum Mode { kF16 = 0, kF16W = 1, kI8 = 2, kI8Norm = 3, kI8Silu = 4, kI8Quant = 5, kF16Norm = 6 };

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
    int batch;              // vectors handled by this launch (1..4, FP16 modes)
    int part_q, part_r;     // items = gridDim.x * part_q + part_r; CTA c owns q (+1 if c < r) items
    int aligned;            // 1: items are whole row blocks (no block spans two CTAs); 0: items are tiles
    int late_release;       // 1: the next kernel in the stream is released after this kernel's own dependency
                            //    wait instead of at its start (see release_rule)
    int ring_slots;         // R
    int l2_prefetch;        // 1: warps prefetch into L2 the chunks beyond what the ring holds
    int ksplit;             // 1 = clusters of two CTAs share whole row blocks, each CTA contracting one half of
                            // the columns (and staging only that half of the activations); the halves' sums
                            // meet in the shared memory of the cluster's first CTA.  part_q/part_r then
                            // partition the row blocks over the clusters
    int off_pairbuf;        // shared memory: float [2][row blocks of the cluster][16] of that exchange
    int pair;               // FP16 modes: 1 = launched as clusters of two CTAs that stage half of the activations
                            // each and write their digits into both CTAs' shared memory
    int x_local;            // FP16 modes, CTAs with fewer tiles than a row has groups: a CTA stages only
                            // the groups it walks (a cyclic run starting at its first tile's group)
    uint2* ws;              // [gridDim.x][2][ws_stride / 2] partial records {value, flag} of this ticket,
                            // all zero between launches
    int ws_stride;          // words per CTA in ws (two records)
    int* err;               // device error flag (0 = none)
    // shared memory carve-up (byte offsets); the staged activations start at 0
    int off_xcst, off_part, off_mask, off_ring, off_bar;
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
// stream-order wait over, activations staged, last tile done, partial sums exchanged
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
// One chunk (n16 pieces of 16 bytes: 34 per tile) global -> shared by the 32 lanes of a warp,
// then each lane makes the slot's mbarrier count its copies: the barrier (initialised to 32
// arrivals) completes its phase when every lane's copies have landed.
__device__ __forceinline__ void fill_slot(uint32_t d, const uint8_t* s, uint32_t bar, int lane, int n16)
{
    // d, s: this lane's first piece (slot or chunk start + 16 * lane)
    constexpr int kFull = kSlotBytes / 16;                 // pieces of a whole chunk
    constexpr int kRounds = (kFull + 31) / 32;
    if (n16 == kFull) {                                    // whole chunk: no bounds test but in the last round
#pragma unroll
        for (int i = 0; i < kRounds; i++)
            if ((i + 1) * 32 <= kFull || i * 32 + lane < kFull)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d + i * 512u), "l"(s + i * 512) : "memory");
    } else {
#pragma unroll
        for (int i = 0; i < kRounds; i++)
            if (i * 32 + lane < n16)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d + i * 512u), "l"(s + i * 512) : "memory");
    }
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// Cluster of two CTAs: rank of this CTA, the partner's address of one of my shared-memory
// addresses, a 32-bit store there, and the cluster-wide barrier (every thread of both CTAs).
__device__ __forceinline__ uint32_t cluster_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t peer_addr(uint32_t local, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_peer(uint32_t addr, uint32_t v)
{
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_barrier()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Shared-memory loads by 32-bit shared address.
__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ half2 u32_as_half2(uint32_t v) { return *reinterpret_cast<half2*>(&v); }

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
// The n tiles of a CTA over its warps: warp w owns [warp_start(w), warp_start(w + 1)), about
// n/kWarps tiles each; with eight or more tiles per warp the starts are rounded down to whole
// chunks, so that chunks and row blocks (of a multiple of four groups) stay aligned.
__device__ __forceinline__ int warp_start(int w, int n)
{
    const int s = (w * n) >> kWarpsLog2;
    return (n >= 8 * kWarps && w < kWarps) ? (s & ~(kSlotTiles - 1)) : s;
}

// ---------------------------------------------------------------------------
// Activation staging
// ---------------------------------------------------------------------------
// Shared-memory layout of the staged activations, FP16 modes.  NB = MMA column blocks
// (n8) per operand register, NV = vectors per block (1 or 2).  Vector v lives in block
// beta = v >> 1 when NV == 2 (beta = 0 when NV == 1), column group vl = v & 1, so that the
// digit d of vector v is B column 4*vl + d of block beta.
//   xdig : uint4 [groups][2 step pairs][NB][NV*4 columns][4 lanes t]
//          the four words of an entry are (b0,b1) of k32 step 2p and (b0,b1) of step 2p+1 of
//          MMA lane (column, t), so one 128-bit shared load feeds two k32 steps; the words of
//          the even step hold 4 x digit;
//   xcst : uint4 [groups][NB*NV]  = {f/64, 64 S_lo, 64 f, 64 S_hi}: f = 2^(e-22) of the group (NaN for
//          a group that holds a non-finite value), S_lo = sum(d0 + 64 d1), S_hi = sum(d2 + 64 d3);
//          lanes of the columns (d0,d1) use the first pair, lanes of (d2,d3) -- worth 4096 -- the
//          second; the 64 is the factor the combined MMA results carry.
constexpr uint32_t kDigitOffset = 32u * (1u + 64u + 4096u + 262144u);    // 8521760

// Digit words of four consecutive activations u0..u3 (each q + kDigitOffset, 24 bits): byte k
// of word i is the 6-bit digit i of activation k as a signed byte, shifted left by `sh` (0 or
// 2: the even k32 steps carry 4 x digit).  The bytes of the four values are transposed first,
// so that every mask and shift then works on four activations at once.
__device__ __forceinline__ void quad_digits(uint32_t u0, uint32_t u1, uint32_t u2, uint32_t u3, uint32_t sh, uint32_t bias,
                                            uint32_t (&w)[4])
{
    const uint32_t a = __byte_perm(u0, u1, 0x5140), b = __byte_perm(u2, u3, 0x5140);
    const uint32_t c = __byte_perm(u0, u1, 0x0062), d = __byte_perm(u2, u3, 0x0062);
    const uint32_t t0 = __byte_perm(a, b, 0x5410);          // bits  0..7  of the four values
    const uint32_t t1 = __byte_perm(a, b, 0x7632);          // bits  8..15
    const uint32_t t2 = __byte_perm(c, d, 0x5410);          // bits 16..23
    uint32_t v[4];
    v[0] = t0 & 0x3f3f3f3fu;
    v[1] = ((t0 >> 6) & 0x03030303u) | ((t1 << 2) & 0x3c3c3c3cu);
    v[2] = ((t1 >> 4) & 0x0f0f0f0fu) | ((t2 << 4) & 0x30303030u);
    v[3] = (t2 >> 2) & 0x3f3f3f3fu;
    // field v in 0..63 -> (v - 32) or 4 (v - 32) as a signed byte: bias = 0x60606060 or 0
#pragma unroll
    for (int i = 0; i < 4; i++) w[i] = ((v[i] << sh) + bias) ^ 0x80808080u;
}

// Each thread converts 8 consecutive activations (one 128-bit load); the 16 lanes of a
// half-warp cover one scale group and agree on its exponent and sums with shuffles.
// The groups staged are the cyclic run g0, g0+1, ... (mod groups) of length gcount; staged
// group number i of that run is stored at index i (gcount == groups, g0 == 0: all of them).
// part / nparts / peer: with nparts == 2 this CTA converts every second batch of kThreads items
// (those of parity `part`) and stores each result word to its own shared memory and, at `peer`
// (the partner's address of xdig; the constants follow at the same distance), to the partner's.
// SMEM_SRC: x is a vector in shared memory (made by norm_to_smem), read with plain loads.
template <int NB, int NV, bool SMEM_SRC = false>
__device__ __forceinline__ void stage_x_f16(const half* __restrict__ x, int cols, int groups, int batch,
                                            uint32_t* xdig, uint4* xcst, int tid, int g0, int gcount,
                                            int part = 0, int nparts = 1, uint32_t peer = 0)
{
    constexpr int NVT = NB * NV;
    const int per_vec = gcount << 4;               // 8-element items per vector (16 per group)
    const int items = per_vec * batch;             // a multiple of 16: a half-warp is all in or all out
    const int l16 = tid & 15;
    // vectors of the last block that do not exist: their constants are zero, so whatever the
    // MMA makes of their (unwritten) digit columns never reaches a finite-times-NaN product
    if (NVT > 1)
        for (int i = tid; i < gcount * (NVT - batch); i += kThreads) {
            const int g = i / (NVT - batch), v = batch + i % (NVT - batch);
            xcst[g * NVT + v] = make_uint4(0u, 0u, 0u, 0u);
        }
    // elements 8*l16 .. 8*l16+7 of a group: k32 step m = l16 / 4, half j2 = (l16 / 2) & 1,
    // MMA lanes t = 2*(l16 & 1) and the next one; the even steps carry 4 x digit
    const int m = l16 >> 2, j2 = (l16 >> 1) & 1, t0 = 2 * (l16 & 1);
    const uint32_t sh = (m & 1) ? 0u : 2u, bias = (m & 1) ? 0x60606060u : 0u;
    const int lane_off = t0 * 4 + (m & 1) * 2 + j2 + (m >> 1) * (NB * NV * 64);   // words, inside a group's entry
    auto fetch = [&](int item) {
        const int b = (NVT == 1) ? 0 : (int)((unsigned)item / (unsigned)per_vec);
        const int el = item - b * per_vec;
        int gg = g0 + (el >> 4);
        if (gg >= groups) gg -= groups;
        const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)b * cols) + (gg << 4) + l16;
        if (SMEM_SRC) return *src;
        return __ldg(src);
    };
    const int stride = kThreads * nparts;
    int item = tid + part * kThreads;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (item < items) raw = fetch(item);
    for (; (item & ~31) < items; item += stride) {            // warp-uniform: the shuffles need every lane
        const bool valid = item < items;
        const uint4 cur = raw;
        if (item + stride < items) raw = fetch(item + stride);          // in flight during this item's arithmetic
        const int b = (NVT == 1 || !valid) ? 0 : (int)((unsigned)item / (unsigned)per_vec);
        const int g = ((valid ? item : 0) - b * per_vec) >> 4;          // staged group number
        // largest magnitude of the group as an FP16 bit pattern: orders finite values,
        // infinities and NaNs alike
        uint32_t mb = __vmaxu2(__vmaxu2(cur.x & 0x7fff7fffu, cur.y & 0x7fff7fffu),
                               __vmaxu2(cur.z & 0x7fff7fffu, cur.w & 0x7fff7fffu));
        mb = max(mb & 0xffffu, mb >> 16);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, o));
        const bool finite = mb < 0x7c00u;
        const bool live = finite && mb != 0u;
        // 2^e > max|x| with e = E - 14 (E the biased FP16 exponent; subnormals count as E = 1)
        const int e = (int)max(mb >> 10, 1u) - 14;
        const float up = live ? __uint_as_float((uint32_t)(22 - e + 127) << 23) : 0.f;
        const float dn = finite ? (mb != 0u ? __uint_as_float((uint32_t)(e - 22 + 127) << 23) : 0.f)
                                : __uint_as_float(0x7fc00000u);
        // q = rint(x * up) through the mantissa of x * up + 1.5 * 2^23 (one rounding, to nearest even,
        // |q| < 2^22), and u = q + kDigitOffset
        uint32_t u[8];
        {
            const uint32_t rw[4] = {cur.x, cur.y, cur.z, cur.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 f = __half22float2(*reinterpret_cast<const half2*>(&rw[i]));
                u[2 * i] = __float_as_uint(fmaf(f.x, up, 12582912.0f)) - 0x4b400000u + kDigitOffset;
                u[2 * i + 1] = __float_as_uint(fmaf(f.y, up, 12582912.0f)) - 0x4b400000u + kDigitOffset;
            }
        }
        uint32_t w[2][4];
        quad_digits(u[0], u[1], u[2], u[3], sh, bias, w[0]);
        quad_digits(u[4], u[5], u[6], u[7], sh, bias, w[1]);
        // digit sums of the group (times 4 on the even steps): low pair d0 + 64 d1, high pair d2 + 64 d3
        int sd[4];
#pragma unroll
        for (int d = 0; d < 4; d++) sd[d] = __dp4a((int)w[1][d], 0x01010101, __dp4a((int)w[0][d], 0x01010101, 0));
        int slo = (sd[0] + 64 * sd[1]) >> sh, shi = (sd[2] + 64 * sd[3]) >> sh;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            slo += __shfl_xor_sync(0xffffffffu, slo, o);
            shi += __shfl_xor_sync(0xffffffffu, shi, o);
        }
        if (valid) {
            const int beta = (NV == 2) ? (b >> 1) : 0, vl = (NV == 2) ? (b & 1) : 0;
            const int pw = ((g * 2 * NB + beta) * (NV * 4) + vl * 4) * 16 + lane_off;
            uint32_t* p = xdig + pw;
#pragma unroll
            for (int h = 0; h < 2; h++)             // second quad: next lane t
#pragma unroll
                for (int d = 0; d < 4; d++) {
                    p[(d * 4 + h) * 4] = w[h][d];
                    if (nparts > 1) st_peer(peer + (uint32_t)(pw + (d * 4 + h) * 4) * 4u, w[h][d]);
                }
            if (l16 == 0) {
                const uint4 c = make_uint4(__float_as_uint(dn * 0.015625f), (uint32_t)(slo * 64),
                                           __float_as_uint(dn * 64.0f), (uint32_t)(shi * 64));
                xcst[g * NVT + b] = c;
                if (nparts > 1) {
                    const uint32_t pc = peer + (uint32_t)(reinterpret_cast<uint8_t*>(xcst + g * NVT + b) - reinterpret_cast<uint8_t*>(xdig));
                    st_peer(pc, c.x);
                    st_peer(pc + 4, c.y);
                    st_peer(pc + 8, c.z);
                    st_peer(pc + 12, c.w);
                }
            }
        }
    }
}

// kF16W staging: 16-bit block fixed point, q = rint(x * 2^(15-e)) = d0 + 256 d1 with both digits
// signed bytes (q in [-32896, 32639]: a group whose largest magnitude is within 0.8 % of the
// next power of two takes one exponent more), four vectors per column block, no pre-scaled
// steps.  The rounding error per element is at most 2^-17 of the group's largest magnitude:
// 128 * 2^-17 = 1e-3 of it per group, half of the 2e-3 * sum|scale * x| the benchmark allows
// even if every other activation of the group were zero.
//   xdig : uint4 [groups][2 step pairs][NB][8 columns = 4 vectors x 2 digits][4 lanes t]
//   xcst : uint4 [groups][4 NB] = {f/64, 64 S, 0, 0}, f = 2^(e-15), S = sum(q)
template <int NB>
__device__ __forceinline__ void stage_x_f16w(const half* __restrict__ x, int cols, int groups, int batch,
                                             uint32_t* xdig, uint4* xcst, int tid, int g0, int gcount,
                                             int part = 0, int nparts = 1, uint32_t peer = 0)
{
    constexpr int NVT = NB * 4;
    const int per_vec = gcount << 4;
    const int items = per_vec * batch;
    const int l16 = tid & 15;
    for (int i = tid; i < gcount * (NVT - batch); i += kThreads) {
        const int g = i / (NVT - batch), v = batch + i % (NVT - batch);
        xcst[g * NVT + v] = make_uint4(0u, 0u, 0u, 0u);
    }
    const int m = l16 >> 2, j2 = (l16 >> 1) & 1, t0 = 2 * (l16 & 1);
    const int lane_off = t0 * 4 + (m & 1) * 2 + j2 + (m >> 1) * (NB * 8 * 16);     // words, inside a group's entry
    auto fetch = [&](int item) {
        const int b = (int)((unsigned)item / (unsigned)per_vec);
        const int el = item - b * per_vec;
        int gg = g0 + (el >> 4);
        if (gg >= groups) gg -= groups;
        return __ldg(reinterpret_cast<const uint4*>(x + (size_t)b * cols) + (gg << 4) + l16);
    };
    const int stride = kThreads * nparts;
    int item = tid + part * kThreads;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (item < items) raw = fetch(item);
    for (; (item & ~31) < items; item += stride) {
        const bool valid = item < items;
        const uint4 cur = raw;
        if (item + stride < items) raw = fetch(item + stride);
        const int b = valid ? (int)((unsigned)item / (unsigned)per_vec) : 0;
        const int g = ((valid ? item : 0) - b * per_vec) >> 4;
        uint32_t mb = __vmaxu2(__vmaxu2(cur.x & 0x7fff7fffu, cur.y & 0x7fff7fffu),
                               __vmaxu2(cur.z & 0x7fff7fffu, cur.w & 0x7fff7fffu));
        mb = max(mb & 0xffffu, mb >> 16);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, o));
        const bool finite = mb < 0x7c00u;
        const bool live = finite && mb != 0u;
        const int e = (int)max(mb >> 10, 1u) - 14 + ((mb & 0x3ffu) >= 1016u ? 1 : 0);
        const float up = live ? __uint_as_float((uint32_t)(15 - e + 127) << 23) : 0.f;
        const float dn = finite ? (mb != 0u ? __uint_as_float((uint32_t)(e - 15 + 127) << 23) : 0.f)
                                : __uint_as_float(0x7fc00000u);
        // u = q + 32896: its two bytes are the digits plus 128
        uint32_t u[8];
        {
            const uint32_t rw[4] = {cur.x, cur.y, cur.z, cur.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 f = __half22float2(*reinterpret_cast<const half2*>(&rw[i]));
                u[2 * i] = __float_as_uint(fmaf(f.x, up, 12582912.0f)) - 0x4b400000u + 32896u;
                u[2 * i + 1] = __float_as_uint(fmaf(f.y, up, 12582912.0f)) - 0x4b400000u + 32896u;
            }
        }
        uint32_t w[2][2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t a = __byte_perm(u[4 * h], u[4 * h + 1], 0x5140), c = __byte_perm(u[4 * h + 2], u[4 * h + 3], 0x5140);
            w[h][0] = __byte_perm(a, c, 0x5410) ^ 0x80808080u;
            w[h][1] = __byte_perm(a, c, 0x7632) ^ 0x80808080u;
        }
        int sq = __dp4a((int)w[1][0], 0x01010101, __dp4a((int)w[0][0], 0x01010101, 0)) +
                 256 * __dp4a((int)w[1][1], 0x01010101, __dp4a((int)w[0][1], 0x01010101, 0));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (valid) {
            const int beta = b >> 2, vl = b & 3;
            const int pw = ((g * 2 * NB + beta) * 8 + vl * 2) * 16 + lane_off;
            uint32_t* p = xdig + pw;
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int d = 0; d < 2; d++) {
                    p[(d * 4 + h) * 4] = w[h][d];
                    if (nparts > 1) st_peer(peer + (uint32_t)(pw + (d * 4 + h) * 4) * 4u, w[h][d]);
                }
            if (l16 == 0) {
                const uint32_t c0 = __float_as_uint(dn * 0.015625f), c1 = (uint32_t)(sq * 64);
                xcst[g * NVT + b] = make_uint4(c0, c1, 0u, 0u);
                if (nparts > 1) {
                    const uint32_t pc = peer + (uint32_t)(reinterpret_cast<uint8_t*>(xcst + g * NVT + b) - reinterpret_cast<uint8_t*>(xdig));
                    st_peer(pc, c0);
                    st_peer(pc + 4, c1);
                }
            }
        }
    }
}

// INT8 activations in shared memory: two digit columns, x = lo + 16 hi with lo = x & 15 (0..15)
// and hi = x >> 4 (-8..7), laid out like the FP16 digits: uint4 [groups][2 step pairs][2 columns]
// [4 lanes t], words (b0,b1) of step 2p and (b0,b1) of step 2p+1, the even step times 4.
// Stores the two digit words of original word w of the vector (four consecutive activations).
__device__ __forceinline__ void store_i8_word(uint32_t* xq, int w, uint32_t xw)
{
    const int g = w >> 5, r = w & 31;
    const int m = r >> 3, j2 = (r >> 2) & 1, t = r & 3;
    uint32_t lo = xw & 0x0f0f0f0fu;
    const uint32_t h = (xw >> 4) & 0x0f0f0f0fu;
    uint32_t hi = h | ((h & 0x08080808u) * 0x1eu);           // sign-extend each nibble to a byte
    if ((m & 1) == 0) {
        lo <<= 2;
        hi = (hi << 2) & 0xfcfcfcfcu;
    }
    uint32_t* p = xq + (((g * 2 + (m >> 1)) * 2) * 4 + t) * 4 + (m & 1) * 2 + j2;
    p[0] = lo;
    p[16] = hi;
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

// INT8 vector from global memory: its digit columns plus 64 x the per-group sums, sx[groups] (64
// is the factor the combined MMA results carry).
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
            store_i8_word(xq, 4 * i, v.x);
            store_i8_word(xq, 4 * i + 1, v.y);
            store_i8_word(xq, 4 * i + 2, v.z);
            store_i8_word(xq, 4 * i + 3, v.w);
            if ((i & 7) == 0) sx[i >> 3] = s * 64;
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
// tmp[cols] (shared memory) = FP16(rmsnorm(a (+ b)) * w), the arithmetic of the stand-alone
// rmsnorm operator: FP16-rounded sum first (stored to res_out by CTA 0 when a and b are both
// given), mean of squares and scaling in FP32, one FP16 rounding of the result.  Every CTA of
// the GEMV computes the whole vector (the inputs are a few KB in L2).  Ends with a barrier.
__device__ __forceinline__ void norm_to_smem(const GemvArgs& a, half* tmp, float* red, int tid)
{
    const int n8 = a.cols >> 3;
    float ss = 0.f;
    for (int i = tid; i < n8; i += kThreads) {
        const uint4 ar = *(reinterpret_cast<const uint4*>(a.fx_a) + i);
        uint4 st4 = ar;
        if (a.fx_b) {
            const uint4 br = *(reinterpret_cast<const uint4*>(a.fx_b) + i);
            const half* ah = reinterpret_cast<const half*>(&ar);
            const half* bh = reinterpret_cast<const half*>(&br);
            half* sth = reinterpret_cast<half*>(&st4);
#pragma unroll
            for (int j = 0; j < 8; j++) sth[j] = __float2half_rn(__half2float(ah[j]) + __half2float(bh[j]));
            if (a.fx_res_out && blockIdx.x == 0) *(reinterpret_cast<uint4*>(a.fx_res_out) + i) = st4;
        }
        const half* vh = reinterpret_cast<const half*>(&st4);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float v = __half2float(vh[j]);
            ss += v * v;
        }
        *(reinterpret_cast<uint4*>(tmp) + i) = st4;
    }
    const float var = cta_sum(ss, red, tid) / (float)a.cols;
    const float rinv = rsqrtf(var + a.fx_eps);
    for (int i = tid; i < n8; i += kThreads) {
        uint4 v4 = *(reinterpret_cast<const uint4*>(tmp) + i);
        const uint4 w4 = __ldg(reinterpret_cast<const uint4*>(a.fx_w) + i);
        half* vh = reinterpret_cast<half*>(&v4);
        const half* wh = reinterpret_cast<const half*>(&w4);
#pragma unroll
        for (int j = 0; j < 8; j++) vh[j] = __float2half_rn(__half2float(vh[j]) * rinv * __half2float(wh[j]));
        *(reinterpret_cast<uint4*>(tmp) + i) = v4;
    }
    __syncthreads();
}

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
            store_i8_word(xq, 2 * i, w[0]);
            store_i8_word(xq, 2 * i + 1, w[1]);
            if ((i & 15) == 0) sx[i >> 4] = s * 64;
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
// KS: the column split inside clusters of two CTAs (GemvArgs::ksplit), an instantiation of its own
// so that the other launches carry none of its bookkeeping.
template <int MODE, int NB, int NV, bool AR, bool KS = false>
__global__ void __launch_bounds__(kThreads, 2) gemv_packed_kernel(const __grid_constant__ GemvArgs a)
{
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr bool FUSEDX = (MODE == kI8Norm || MODE == kI8Silu || MODE == kI8Quant);
    constexpr bool I8 = (MODE == kI8 || FUSEDX);
    constexpr bool W16 = (MODE == kF16W);         // four vectors per column block, two 8-bit digits each
    constexpr bool F16N = (MODE == kF16Norm);     // FP16 digits of a vector normalised in the staging phase
    constexpr int NVT = NB * NV;                  // vectors per weight pass
    static_assert(!I8 || (NB == 1 && NV == 1), "INT8 modes carry one vector");
    static_assert(!W16 || NV == 4, "the wide FP16 mode carries four vectors per column block");

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
#ifdef TLLM_TIMELINE
    if (threadIdx.x == 0)
        g_tl[tl_slot][blockIdx.x][7] = (unsigned long long)a.aligned | ((unsigned long long)a.ring_slots << 8) |
                                       ((unsigned long long)gridDim.x << 20) | ((unsigned long long)a.part_q << 32);
#endif
    // Kernel parameters sit in a constant bank that is new with every launch: the first read of
    // each of its cache lines goes out to memory.  Every line is read once here, where the
    // latency hides behind the previous kernel, and the part of the kernel that runs after the
    // last tile -- on the critical path of the stream -- reads the copy in shared memory.
    __shared__ __align__(16) uint32_t sargs[(sizeof(GemvArgs) + 3) / 4];
    if (tid < (int)(sizeof(GemvArgs) / 4)) sargs[tid] = reinterpret_cast<const uint32_t*>(&a)[tid];
    const int G = a.groups, R = a.ring_slots;
    // Column split inside a cluster of two CTAs (FP16, one vector): the partition items are the
    // clusters' row blocks; this CTA walks, for each of them, the run of G/2 tiles of its half.
    static_assert(!KS || (MODE == kF16 && NB == 1 && NV == 1), "the column split carries one FP16 vector");
    constexpr bool ksplit = KS;
    const int krank = ksplit ? (int)(blockIdx.x & 1u) : 0;               // = %cluster_ctarank (clusters along x)
    const int pid = ksplit ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;   // partition index: cluster or CTA
    const int run = ksplit ? (G >> 1) : G;                                 // tiles this CTA walks per row block
    const int per = a.aligned ? run : 1;                                   // tiles per partition item
    // first tile of this CTA in memory, and its tiles (for ksplit: in runs of `run`, G apart)
    const int t0 = part_start(pid, a.part_q, a.part_r) * (a.aligned ? G : 1) + krank * run;
    const int n = (a.part_q + (pid < a.part_r ? 1 : 0)) * per;
    // first and last row block this CTA holds tiles of (whole row blocks: no division needed)
    const int rb_first = a.aligned ? part_start(pid, a.part_q, a.part_r) : (int)((unsigned)t0 / (unsigned)G);
    const int rb_last = a.aligned ? rb_first + a.part_q - (pid < a.part_r ? 0 : 1)
                                  : (int)((unsigned)(t0 + n - 1) / (unsigned)G);

    uint32_t* xstage = reinterpret_cast<uint32_t*>(smem);              // digits, or the int8 vector
    uint4* xcst = reinterpret_cast<uint4*>(smem + a.off_xcst);         // FP16 modes: group constants
    int* sx = reinterpret_cast<int*>(smem + a.off_xcst);               // INT8 modes: 64 x group sums
    float* part = reinterpret_cast<float*>(smem + a.off_part);         // [segment][16 rows][NVT]
    uint32_t* contrib = reinterpret_cast<uint32_t*>(smem + a.off_mask);    // per row block of this CTA: the warps that hold sums of it
    const uint32_t ring = smem_addr(smem + a.off_ring);
    const uint32_t bar = smem_addr(smem + a.off_bar);

    // ---- this warp's tile range, in chunks of four, and the first ring fill ------------
    // v0: this warp's first tile counted along the CTA's walk; w0: the same tile in memory (with
    // ksplit the walk skips the other CTA's half of every row block)
    const int v0 = warp_start(warp, n), nw = warp_start(warp + 1, n) - v0;   // nw may be 0 for tiny problems
    const int vrb = ksplit ? (int)((unsigned)v0 / (unsigned)run) : 0;       // row blocks in front of v0 (ksplit)
    const int w0 = t0 + v0 + (ksplit ? vrb * (G - run) : 0);
    const int nchunks = (nw + kSlotTiles - 1) / kSlotTiles;
    // this warp's private ring: slots s0 .. s0 + depth - 1 of the CTA's R
    const int depth = (R >> kWarpsLog2) + (warp < (R & (kWarps - 1)) ? 1 : 0);
    const int s0 = warp * (R >> kWarpsLog2) + min(warp, R & (kWarps - 1));
    const uint32_t ring_w = ring + (uint32_t)s0 * kSlotBytes + (uint32_t)lane * 16u;   // this lane's first piece of slot 0
    const uint32_t bar_w = bar + (uint32_t)s0 * 8u;
    if (lane == 0) {
        for (int k = 0; k < depth; k++) mbar_init(bar_w + k * 8, 32);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    // pieces of 16 bytes in chunk c of this warp's range
    auto pieces = [&](int c) { return min(kSlotTiles, nw - c * kSlotTiles) * (kTileBytes / 16); };
    const uint8_t* src_lane = a.packed + (size_t)w0 * kTileBytes + (size_t)lane * 16;
    // chunk `cidx` of this warp's range -> L2, one 128-byte line per lane
    auto l2_chunk = [&](int cidx) {
        const uint8_t* p0 = a.packed + (size_t)(w0 + cidx * kSlotTiles) * kTileBytes;
        const uint32_t bytes = (uint32_t)min(kSlotTiles, nw - cidx * kSlotTiles) * kTileBytes;
        const uintptr_t first = reinterpret_cast<uintptr_t>(p0) & ~(uintptr_t)127;
        const uint32_t lines = (uint32_t)((reinterpret_cast<uintptr_t>(p0) + bytes - first + 127) >> 7);
        if ((uint32_t)lane < lines) asm volatile("prefetch.global.L2 [%0];" ::"l"(first + (uintptr_t)lane * 128) : "memory");
    };
    const int cinit = min(depth, nchunks);                   // chunks of the first ring fill
    // the request stream: next chunk's address, and (ksplit) how many tiles of the current run are
    // still to request -- at its end the stream jumps over the other CTA's half.  Chunks never
    // straddle a run: runs and warp ranges are multiples of the chunk (the launch plan sees to it).
    const uint8_t* src_next = src_lane;
    int run_left = ksplit ? run - (v0 - vrb * run) : 0x7fffffff;
    auto advance = [&]() {
        src_next += kSlotBytes;
        if (ksplit) {
            run_left -= kSlotTiles;
            if (run_left <= 0) {
                src_next += (size_t)(G - run) * kTileBytes;
                run_left = run;
            }
        }
    };
    for (int c = 0; c < cinit; c++) {
        fill_slot(ring_w + c * kSlotBytes, src_next, bar_w + c * 8, lane, pieces(c));
        advance();
    }
    if (kL2Ahead > 0 && a.l2_prefetch && !ksplit)
        for (int c = cinit; c < min(nchunks, cinit + kL2Ahead); c++) l2_chunk(c);
    __syncwarp();
    // paired launch: the partner's shared memory may be written once both CTAs are running
    const bool paired = !I8 && !AR && a.pair;
    if (paired || ksplit) cluster_barrier();
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

    for (int i = tid; i <= rb_last - rb_first; i += kThreads) contrib[i] = 0u;    // set in flush(), after the barrier below
    float fused_scale = 1.0f;
    if (FUSEDX) {
        fused_scale = stage_x_fused<MODE>(a, xstage, sx, reinterpret_cast<half*>(smem + a.off_xtmp),
                                          reinterpret_cast<float*>(smem + a.off_xtmp + (size_t)a.cols * sizeof(half)), tid);
    } else if (I8) {
        stage_x_i8(reinterpret_cast<const int8_t*>(a.x), a.cols, xstage, sx, tid);
    } else {
        const int g0 = ksplit ? krank * run : (a.x_local ? (int)((unsigned)t0 % (unsigned)G) : 0);
        const int gstage = ksplit ? run : (a.x_local ? n : G);
        const int part = paired ? (int)cluster_rank() : 0, nparts = paired ? 2 : 1;
        const uint32_t peer = paired ? peer_addr(smem_addr(xstage), (uint32_t)(part ^ 1)) : 0u;
        if constexpr (F16N) {
            half* tmp = reinterpret_cast<half*>(smem + a.off_xtmp);
            norm_to_smem(a, tmp, reinterpret_cast<float*>(smem + a.off_xtmp + (size_t)a.cols * sizeof(half)), tid);
            stage_x_f16<NB, NV, true>(tmp, a.cols, G, 1, xstage, xcst, tid, g0, gstage);
        } else if constexpr (W16)
            stage_x_f16w<NB>(reinterpret_cast<const half*>(a.x), a.cols, G, a.batch, xstage, xcst, tid, g0,
                             gstage, part, nparts, peer);
        else
            stage_x_f16<NB, NV>(reinterpret_cast<const half*>(a.x), a.cols, G, a.batch, xstage, xcst, tid, g0,
                                gstage, part, nparts, peer);
    }
    // both halves of a paired launch are in place (and no store to the partner is outstanding)
    // once every thread of the two CTAs has passed this barrier; it orders the CTA's own
    // shared-memory writes like __syncthreads()
    if (paired)
        cluster_barrier();
    else
        __syncthreads();
    TL(3);

    // ---- per-lane constants ------------------------------------------------------
    const int t = lane & 3, gq = lane >> 2;
    // This lane's accumulator columns 2t, 2t+1 are two digits of one vector.  FP16: digits (0,1)
    // of vector t/2 of the block when t is even, digits (2,3) -- worth 4096 -- when t is odd; the
    // second digit of a pair counts 64.  INT8: (lo, hi) in columns 0, 1, the second counts 16.
    constexpr int kMulA = I8 ? 16 : 64;
    // B operand entry of this lane: column gq -> FP16 (vector gq / 4 of the block, digit gq % 4),
    // INT8 digit gq; lanes of columns that carry nothing read a neighbour's entry, their products
    // are unused.  Shared-memory addresses are kept as 32-bit numbers.
    const int bcol = I8 ? min(gq, 1) : (W16 ? gq : (min(gq >> 2, NV - 1) * 4 + (gq & 3)));
    constexpr int kXbStride = I8 ? 8 : (W16 ? 32 : NV * 16);    // entries per (group, step pair, block)
    constexpr uint32_t kXgBytes = 2u * NB * kXbStride * 16u;    // staged bytes per group
    const uint32_t xb_addr = smem_addr(xstage) + (uint32_t)(bcol * 4 + t) * 16u;
    // group constants of this lane: FP16 {factor, offset} pair (first pair for even t, second for odd)
    const uint32_t xc_addr = smem_addr(smem + a.off_xcst) + ((I8 || W16) ? 0u : (uint32_t)(t & 1) * 8u);
    const uint32_t sc_off = kTileCodeBytes + (uint32_t)gq * 4u;      // this lane's two scales inside a tile
    const bool xloc = !I8 && a.x_local;

    // ---- main loop: this warp's tiles, four per ring slot ----------------------------
    // g: position of the next tile inside this CTA's run of its row block (the group, or with
    // ksplit the group counted from the CTA's first); a run ends at `run`
    const int rb0 = ksplit ? rb_first + vrb : (int)((unsigned)w0 / (unsigned)G);
    int g = ksplit ? v0 - vrb * run : w0 - rb0 * G;
    int gxi = xloc ? v0 : g;                 // where that group's activations were staged
    int rbr = rb0 - rb_first;                // row block, relative to the CTA's first
    float acc[NB][2];                        // [block][row half h]: rows gq + 8h of the row block
#pragma unroll
    for (int b = 0; b < NB; b++) acc[b][0] = acc[b][1] = 0.f;
    bool ok = true;

    // sums of the tiles walked since the last flush -> this warp's record of the row block
    auto flush = [&]() {
        float* pu = part + (size_t)(rbr + warp) * (kTileRows * NVT);     // unique per (warp, row block), ascending
        if (lane == 0) atomicOr(contrib + rbr, 1u << warp);
#pragma unroll
        for (int b = 0; b < NB; b++)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                float v = acc[b][h];
                if (!I8 && !W16) v += __shfl_xor_sync(0xffffffffu, v, 1);   // lanes t, t^1: the digit halves of one vector
                const int row = gq + 8 * h;
                if (I8) {
                    if (t == 0) pu[row] = v;
                } else if (W16) {
                    pu[row * NVT + b * 4 + t] = v;                  // lane t holds vector t of the block
                } else if ((t & 1) == 0 && (t >> 1) < NV) {
                    pu[row * NVT + b * NV + (t >> 1)] = v;
                }
                acc[b][h] = 0.f;
            }
    };

    // One tile at shared address tp, activations of staged group gx: two MMA chains (steps 0,1
    // carry the factor 4; steps 2,3 carry 64), joined in integers, the code offset removed,
    // scale and block exponent applied.
    auto tile = [&](uint32_t tp, int gx) {
        const uint4 wd = lds128(tp + (uint32_t)lane * 16u);
        const float2 sc = __half22float2(u32_as_half2(lds32(tp + sc_off)));
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const uint32_t xa = xb_addr + (uint32_t)gx * kXgBytes + (uint32_t)b * (kXbStride * 16u);
            const uint4 xb0 = lds128(xa);
            const uint4 xb1 = lds128(xa + NB * kXbStride * 16u);
            int p0, p1;
            float fx;
            if constexpr (W16) {
                // four independent MMAs, one per 32-column step; step f carries the factor 4^f of
                // its bit field, so ((D0*4 + D1)*4 + D2)*4 + D3 = 64 * (sum over the group) per
                // column; columns 2t, 2t+1 are the low and the high digit of vector t
                int d0[4], d1[4], d2[4], d3[4];
                imma<true>(d0, wd.x & 0x03030303u, wd.z & 0x03030303u, wd.y & 0x03030303u, wd.w & 0x03030303u, xb0.x, xb0.y);
                imma<true>(d1, wd.x & 0x0c0c0c0cu, wd.z & 0x0c0c0c0cu, wd.y & 0x0c0c0c0cu, wd.w & 0x0c0c0c0cu, xb0.z, xb0.w);
                imma<true>(d2, wd.x & 0x30303030u, wd.z & 0x30303030u, wd.y & 0x30303030u, wd.w & 0x30303030u, xb1.x, xb1.y);
                imma<true>(d3, wd.x & 0xc0c0c0c0u, wd.z & 0xc0c0c0c0u, wd.y & 0xc0c0c0c0u, wd.w & 0xc0c0c0c0u, xb1.z, xb1.w);
                int q[4];
#pragma unroll
                for (int i = 0; i < 4; i++) q[i] = ((d0[i] * 4 + d1[i]) * 4 + d2[i]) * 4 + d3[i];
                const uint2 c = lds64(xc_addr + (uint32_t)(gx * NVT + b * 4 + t) * 16u);
                fx = __uint_as_float(c.x);
                p0 = q[1] * 256 + q[0] - (int)c.y;
                p1 = q[3] * 256 + q[2] - (int)c.y;
            } else {
            int lo[4], hi[4];
            // words (h, j2) = (0,0) (0,1) (1,0) (1,1) are registers a0, a2, a1, a3
            imma<true>(lo, wd.x & 0x03030303u, wd.z & 0x03030303u, wd.y & 0x03030303u, wd.w & 0x03030303u, xb0.x, xb0.y);
            imma<true>(hi, wd.x & 0x30303030u, wd.z & 0x30303030u, wd.y & 0x30303030u, wd.w & 0x30303030u, xb1.x, xb1.y);
            imma<false>(lo, wd.x & 0x0c0c0c0cu, wd.z & 0x0c0c0c0cu, wd.y & 0x0c0c0c0cu, wd.w & 0x0c0c0c0cu, xb0.z, xb0.w);
            imma<false>(hi, wd.x & 0xc0c0c0c0u, wd.z & 0xc0c0c0c0u, wd.y & 0xc0c0c0c0u, wd.w & 0xc0c0c0c0u, xb1.z, xb1.w);
            int soff;
            if (I8) {
                fx = 1.0f;
                soff = (int)lds32(xc_addr + (uint32_t)gx * 4u);
            } else {
                const int v = min(b * NV + (t >> 1), NVT - 1);
                const uint2 c = lds64(xc_addr + (uint32_t)(gx * NVT + v) * 16u);
                fx = __uint_as_float(c.x);
                soff = (int)c.y;
            }
            // lo = 4 * (steps 0,1), hi = 64 * (steps 2,3): lo * 16 + hi = 64 * (sum of the group) per column
            p0 = (lo[1] * 16 + hi[1]) * kMulA + (lo[0] * 16 + hi[0]) - soff;
            p1 = (lo[3] * 16 + hi[3]) * kMulA + (lo[2] * 16 + hi[2]) - soff;
            }
            acc[b][0] = fmaf((float)p0, sc.x * fx, acc[b][0]);
            acc[b][1] = fmaf((float)p1, sc.y * fx, acc[b][1]);
        }
    };

    int rem = nw;                            // tiles still to walk
    int req = nw - min(nw, depth * kSlotTiles);      // tiles still to request (after the first fill)
    uint32_t koff = 0, kbar = 0;             // the ring slot that holds the next chunk: byte offset, barrier offset
    const uint32_t kend = (uint32_t)depth * kSlotBytes;
    uint32_t ph = 0;                         // parity of that slot's current use
    while (rem > 0) {
        ok = mbar_wait(bar_w + kbar, ph);
        if (!ok) break;
        const uint32_t chunk = ring_w - (uint32_t)lane * 16u + koff;
        if (rem >= kSlotTiles && g + kSlotTiles <= run) {
            // common case: a whole chunk inside one row block, straight-line code
#pragma unroll
            for (int q = 0; q < kSlotTiles; q++) tile(chunk + q * kTileBytes, gxi + q);
            g += kSlotTiles;
            gxi += kSlotTiles;
            if (g == run) {
                flush();
                g = 0;
                if (!xloc) gxi = 0;
                rbr++;
            }
        } else {
            // ragged chunk (end of the warp's range or a row-block boundary inside it)
            const int nt = min(kSlotTiles, rem);
            for (int q = 0; q < nt; q++) {
                tile(chunk + q * kTileBytes, gxi);
                gxi++;
                if (++g == run) {            // row block finished (for this warp)
                    flush();
                    g = 0;
                    if (!xloc) gxi = 0;
                    rbr++;
                }
            }
        }
        rem -= kSlotTiles;
        if (kL2Ahead > 0 && a.l2_prefetch && !ksplit) {
            const int cnext = (nw - req + kSlotTiles - 1) / kSlotTiles + kL2Ahead;
            if (cnext < nchunks) l2_chunk(cnext);
        }
        // every lane is done with the slot: refill it with this warp's next chunk not yet requested
        __syncwarp();
        if (req > 0) {
            fill_slot(ring_w + koff, src_next, bar_w + kbar, lane, min(kSlotTiles, req) * (kTileBytes / 16));
            advance();
            req -= kSlotTiles;
        }
        koff += kSlotBytes;
        kbar += 8u;
        if (koff == kend) {
            koff = 0;
            kbar = 0;
            ph ^= 1u;
        }
    }
    if (nw > 0 && g != 0) flush();           // tiles walked since the last flush (a flush resets g)
    if (!ok && lane == 0) atomicExch(a.err, TLLM_ERR_TIMEOUT);
    TL(4);
    __syncthreads();
    TL(5);

    // ---- reduction: warps of this CTA, then CTAs, row block by row block -----------
    const GemvArgs& e = *reinterpret_cast<const GemvArgs*>(sargs);     // complete since the barrier after staging
    const int nb = I8 ? 1 : e.batch;
    // INT8 modes: the 1/64 of the combined MMA results rides on the activation scale
    const float oscale = FUSEDX ? fused_scale * 0.015625f
                                : (I8 ? (e.in_scale_dev ? __ldg(e.in_scale_dev) : e.in_scale) * 0.015625f : 1.0f);
    constexpr int kRec = kTileRows * NVT;    // floats of one row block's sums

    if (kAr && e.ar_world > 0) {
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
        const size_t wslot = (size_t)(epar * e.ar_world + e.ar_rank) * e.ar_rows_max;
        float* pb = reinterpret_cast<float*>(smem + e.off_pairbuf);
        const int nrb_cta = rb_last - rb_first + 1;
        if (ksplit) {
            // column split: the two halves of every row block meet in the first CTA's shared
            // memory first (see below); that CTA then takes part in the exchange between ranks
            const uint32_t pb_remote = krank ? peer_addr(smem_addr(pb), 0u) : 0u;
            for (int r_b = rb_first + warp; r_b <= rb_last; r_b += kWarps) {
                if (lane < kTileRows) {
                    float v = 0.f;
                    for (uint32_t mk = contrib[r_b - rb_first]; mk; mk &= mk - 1u)
                        v += part[(size_t)((r_b - rb_first) + (__ffs(mk) - 1)) * kRec + lane];
                    const int slot = (krank * nrb_cta + (r_b - rb_first)) * kTileRows + lane;
                    if (krank)
                        st_peer(pb_remote + (uint32_t)slot * 4u, __float_as_uint(v));
                    else
                        pb[slot] = v;
                }
            }
            cluster_barrier();
            if (krank) {
                if (tid == 0) e.ar_epoch[blockIdx.x] = epoch;      // this CTA's launch counter keeps in step
                return;
            }
        }
        for (int r_b = rb_first + warp; r_b <= rb_last; r_b += kWarps) {
            for (int idx = lane; idx < kTileRows; idx += 32) {
                float s = 0.f;
                if (ksplit) {
                    const int slot = (r_b - rb_first) * kTileRows + idx;
                    s = pb[slot] + pb[nrb_cta * kTileRows + slot];
                } else {
                    for (uint32_t mk = contrib[r_b - rb_first]; mk; mk &= mk - 1u)      // ascending warp order
                        s += part[(size_t)((r_b - rb_first) + (__ffs(mk) - 1)) * kRec + idx];
                }
                const int r = r_b * kTileRows + idx;
                if (r < e.rows) {
                    const uint2 word = make_uint2(__float_as_uint(s), epoch);
#pragma unroll
                    for (int dst_rank = 0; dst_rank < kMaxPeers; dst_rank++) {
                        if (dst_rank < e.ar_world) {
                            uint2* dst = e.ar_recv[dst_rank] + wslot + r;
                            asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(word.x), "r"(word.y) : "memory");
                        }
                    }
                }
            }
        }
        __syncthreads();                     // ar_abort initialised; all stores issued
        if (tracing) ts[3] = globaltimer();
        const int r_lo = rb_first * kTileRows, r_hi = min(e.rows, (rb_last + 1) * kTileRows);
        const uint2* recv = e.ar_recv[e.ar_rank] + (size_t)epar * e.ar_world * e.ar_rows_max;
        const unsigned all = (1u << e.ar_world) - 1u;
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
                        const uint2* src = recv + (size_t)d * e.ar_rows_max + r;
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
                if (d < e.ar_world) v += __uint_as_float(val[d]);      // rank order: the same sum on every rank
            e.y[r] = __float2half_rn(v);
        }
        if (!ok_ar) atomicExch(e.err, TLLM_ERR_TIMEOUT);
        __syncthreads();
        if (tid == 0) e.ar_epoch[blockIdx.x] = epoch;
        if (tracing) {
            ts[4] = globaltimer();
            unsigned long long* rec = e.ar_trace + (size_t)(epoch % (unsigned)e.ar_trace_cap) * 8;
#pragma unroll
            for (int i = 0; i < 5; i++) rec[i] = ts[i];
            rec[5] = epoch;
        }
        return;
    }

    if (ksplit) {
        // ---- the two halves of every row block meet in the first CTA's shared memory: both
        // CTAs put their row-block sums (warp order) into its exchange buffer -- the second CTA
        // through the cluster's shared-memory window --, the cluster barrier orders the stores,
        // and the first CTA adds first half + second half and writes the outputs.
        float* pb = reinterpret_cast<float*>(smem + e.off_pairbuf);
        const int nrb_cta = rb_last - rb_first + 1;
        const uint32_t pb_remote = krank ? peer_addr(smem_addr(pb), 0u) : 0u;
        for (int r_b = rb_first + warp; r_b <= rb_last; r_b += kWarps) {
            if (lane < kTileRows) {
                float v = 0.f;
                for (uint32_t mk = contrib[r_b - rb_first]; mk; mk &= mk - 1u)     // ascending warp order
                    v += part[(size_t)((r_b - rb_first) + (__ffs(mk) - 1)) * kRec + lane];
                const int slot = (krank * nrb_cta + (r_b - rb_first)) * kTileRows + lane;
                if (krank)
                    st_peer(pb_remote + (uint32_t)slot * 4u, __float_as_uint(v));
                else
                    pb[slot] = v;
            }
        }
        cluster_barrier();
        if (krank == 0) {
            for (int r_b = rb_first + warp; r_b <= rb_last; r_b += kWarps) {
                const int r = r_b * kTileRows + lane;
                if (lane < kTileRows && r < e.rows) {
                    const int slot = (r_b - rb_first) * kTileRows + lane;
                    *out_ptr(e, 0, r) = __float2half_rn((pb[slot] + pb[nrb_cta * kTileRows + slot]) * oscale);
                }
            }
        }
        TL(6);
        return;
    }

    uint2* myrec = e.ws + (size_t)blockIdx.x * e.ws_stride;
    const int rec1 = e.ws_stride >> 1;        // offset of a CTA's second record
    constexpr int kW = (kRec + 31) / 32;      // words per lane in one record (kRec = 16, 32 or 64)
    constexpr int kChunk = 4 / kW;            // records polled together
    const bool mine = (kRec >= 32) || lane < kRec;      // this lane holds a word of the record
    bool ok_c = true;
    for (int r_b = rb_first + warp; r_b <= rb_last; r_b += kWarps) {
        const int ta = max(t0, r_b * G), tb = min(t0 + n, (r_b + 1) * G);     // this CTA's tiles of the block
        const bool full = (tb - ta == G);
        const uint32_t mk0 = contrib[r_b - rb_first];
        float s[kW];
#pragma unroll
        for (int i = 0; i < kW; i++) {
            const int idx = lane + 32 * i;
            float v = 0.f;
            if (mine)
                for (uint32_t mk = mk0; mk; mk &= mk - 1u)                     // ascending warp order
                    v += part[(size_t)((r_b - rb_first) + (__ffs(mk) - 1)) * kRec + idx];
            s[i] = v;
        }
        if (!full) {
            // This row block is shared with neighbouring CTAs (K is split across them).  All but
            // the last of them publish their sums and are done; the last gathers.
            const int c_a = part_of(r_b * G, e.part_q, e.part_r);
            const int c_b = part_of((r_b + 1) * G - 1, e.part_q, e.part_r);
            if ((int)blockIdx.x != c_b) {
                uint2* rec = myrec + ((r_b == rb_first) ? 0 : rec1);
                if (mine) {
#pragma unroll
                    for (int i = 0; i < kW; i++)
                        asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1, %2};"
                                     ::"l"(rec + lane + 32 * i), "r"(__float_as_uint(s[i])), "r"(1u) : "memory");
                }
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
                    const int c_rb = (int)((unsigned)part_start(c, e.part_q, e.part_r) / (unsigned)G);
                    rec[cc] = e.ws + (size_t)c * e.ws_stride + ((r_b == c_rb) ? 0 : rec1) + lane;
                    if (c0 + cc < c_b && mine) pending |= ((1u << kW) - 1u) << (cc * kW);
#pragma unroll
                    for (int i = 0; i < kW; i++) val[cc][i] = 0u;
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
                    if (c0 + cc < c_b && mine) {
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
        if (mine) {
#pragma unroll
            for (int i = 0; i < kW; i++) {
                const int idx = lane + 32 * i;
                const int r = r_b * kTileRows + idx / NVT, b = idx % NVT;
                if (r < e.rows && b < nb) *out_ptr(e, b, r) = __float2half_rn(s[i] * oscale);
            }
        }
    }
    if (!ok_c) atomicExch(e.err, TLLM_ERR_TIMEOUT);
    TL(6);
}

// ---------------------------------------------------------------------------
// Repack: reference layout -> packed layout, and back
// ---------------------------------------------------------------------------
// one thread per code word of the packed matrix; the threads of words (t = 0, j2 = 0) also write
// their row's scale.  Counts sign bits that have no nonzero bit.
__global__ void repack_kernel(const uint32_t* __restrict__ nz, const uint32_t* __restrict__ sg,
                              const half* __restrict__ scales, uint8_t* __restrict__ packed,
                              int rows, int cols, int* __restrict__ noncanon)
{
    const int groups = cols / kGroup, wpr = cols / 32;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long ntiles = (long long)((rows + kTileRows - 1) / kTileRows) * groups;
    if (idx >= ntiles * 128) return;
    const long long tile = idx >> 7;
    const int wi = (int)(idx & 127);
    const int lane = wi >> 2, i = wi & 3;
    const int gq = lane >> 2, t = lane & 3, h = i >> 1, j2 = i & 1;
    const int rb = (int)(tile / groups), g = (int)(tile % groups);
    const int r = rb * kTileRows + gq + 8 * h;
    const int bit0 = 16 * j2 + 4 * t;                       // first of this word's four bits in each mask word
    uint32_t word = 0, stray = 0;
    for (int f = 0; f < 4; f++) {                           // mask word f of the group: columns 32f .. 32f+31
        uint32_t a = 0, s = 0;
        if (r < rows) {
            a = nz[(size_t)r * wpr + g * 4 + f];
            s = sg[(size_t)r * wpr + g * 4 + f];
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
    uint8_t* tp = packed + (size_t)tile * kTileBytes;
    reinterpret_cast<uint32_t*>(tp)[wi] = word;
    if (stray) atomicAdd(noncanon, (int)stray);
    if (t == 0 && j2 == 0)
        reinterpret_cast<half*>(tp + kTileCodeBytes)[tile_scale_index(gq + 8 * h)] =
            (r < rows) ? scales[(size_t)r * groups + g] : __float2half(0.f);
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
    const int g = wd / 4, f = wd % 4;          // mask word wd covers group columns 32f .. 32f+31
    const uint8_t* tp = packed + ((size_t)(r / kTileRows) * groups + g) * kTileBytes;
    const uint32_t* cw = reinterpret_cast<const uint32_t*>(tp);
    const int r16 = r % kTileRows;
    uint32_t a = 0, s = 0;
    for (int c = 0; c < 32; c++) {
        int word, shift;
        tile_locate(r16, 32 * f + c, word, shift);
        const uint32_t code = (cw[word] >> shift) & 3u;
        if (code != 1u) a |= 1u << c;
        if (code == 2u) s |= 1u << c;
    }
    nz[idx] = a;
    sg[idx] = s;
    if (f == 0) scales[(size_t)r * groups + g] = reinterpret_cast<const half*>(tp + kTileCodeBytes)[tile_scale_index(r16)];
}

// ---------------------------------------------------------------------------
// Host side: scratch, registry, launch
// ---------------------------------------------------------------------------
constexpr int kMaxRowBlocks = 1 << 18;          // rows up to 4,194,304
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
    return (size_t)((rows + kTileRows - 1) / kTileRows) * (size_t)(cols / kGroup) * kTileBytes;
}

int packed_row_align() { return kTileRows; }

// Partition of the matrix over CTAs and the shared-memory layout of one launch; the same for
// every entry point (regular, no-allocation, fused all-reduce), which differ only in where the
// cross-CTA scratch lives.  nvt = vectors per pass as instantiated (1, 2 or 4), nvx = vector
// columns stored per group (NB * NV * 3 digit columns), force_aligned: whole row blocks per
// CTA or fail (the fused all-reduce needs it).
static int plan_gemv(GemvArgs& a, int sms, int mode, int nvt, int max_ctas, bool force_aligned, int* grid_out,
                     size_t* smem_out, bool allow_clusters = false)
{
    const int rows = a.rows, cols = a.cols;
    a.groups = cols / kGroup;
    const int nrb = (rows + kTileRows - 1) / kTileRows;
    if (nrb > kMaxRowBlocks) return fail(TLLM_ERR_SHAPE, "rows=%d exceeds %d", rows, kMaxRowBlocks * kTileRows);
    if ((long long)nrb * a.groups >= (1ll << 27))
        return fail(TLLM_ERR_SHAPE, "rows=%d cols=%d: more than 2^27 tiles", rows, cols);
    const int tiles = nrb * a.groups;
    const int grid_max = sms < max_ctas ? sms : max_ctas;
    const bool fusedx = (mode == kI8Norm || mode == kI8Silu || mode == kI8Quant);
    const bool i8 = (mode == kI8 || fusedx);
    const int per_cta_rb = (nrb + grid_max - 1) / grid_max;

    // Shared-memory layout for one way of cutting the matrix: activations | group constants |
    // partial sums | contributor masks | (fused staging) | mbarriers | ring.  Returns the bytes in
    // front of the ring.
    // aligned == 2: whole row blocks per CLUSTER of two CTAs, each CTA one half of the columns
    auto layout = [&](int aligned, int* grid, int* n_max_out) {
        const bool ks = (aligned == 2);
        a.aligned = aligned ? 1 : 0;
        a.ksplit = ks ? 1 : 0;
        const int items = aligned ? nrb : tiles;
        const int parts_max = ks ? grid_max / 2 : grid_max;
        const int parts = items < parts_max ? items : parts_max;
        *grid = ks ? 2 * parts : parts;
        a.part_q = items / parts;
        a.part_r = items % parts;
        const int per = aligned ? (ks ? a.groups / 2 : a.groups) : 1;
        const int n_max = (a.part_q + (a.part_r ? 1 : 0)) * per;    // tiles of the largest CTA
        *n_max_out = n_max;
        a.x_local = (!i8 && !ks && n_max < a.groups) ? 1 : 0;
        const int gstaged = ks ? a.groups / 2 : (a.x_local ? n_max : a.groups);
        // staged activations: INT8 two digit columns; FP16 512 bytes per group and vector on 24
        // bits, 1 KB per group for the four vectors of the wide mode
        size_t off = i8 ? (size_t)cols * 2 : (mode == kF16W ? (size_t)gstaged * 1024 : (size_t)gstaged * nvt * 512);
        off = (off + 15) & ~(size_t)15;
        a.off_xcst = (int)off;
        off += i8 ? (size_t)a.groups * sizeof(int) : (size_t)gstaged * nvt * 16;
        off = (off + 15) & ~(size_t)15;
        a.off_part = (int)off;
        const int max_rb_per_cta = aligned ? (a.part_q + 1) : ((a.part_q + 1 + a.groups - 1) / a.groups + 1);
        off += (size_t)(max_rb_per_cta + kWarps) * kTileRows * nvt * sizeof(float);
        a.off_mask = (int)off;
        off += (size_t)(max_rb_per_cta + 1) * sizeof(uint32_t);
        if (ks) {
            off = (off + 15) & ~(size_t)15;
            a.off_pairbuf = (int)off;
            off += (size_t)2 * max_rb_per_cta * kTileRows * sizeof(float);
        }
        if (fusedx || mode == kF16Norm) {
            off = (off + 15) & ~(size_t)15;
            a.off_xtmp = (int)off;
            off += (size_t)cols * sizeof(half) + 64 * sizeof(float);
        }
        off = (off + 15) & ~(size_t)15;
        a.off_bar = (int)off;
        off += (size_t)kMaxSlots * 8;
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
    // matrix is cut at tile granularity (K is split across CTAs).
    // Chunks (ring slots) a CTA of n tiles walks: every warp rounds its share up to whole chunks.
    auto chunks_of = [](int n) { return kWarps * (((n + kWarps - 1) / kWarps + kSlotTiles - 1) / kSlotTiles); };
    int grid = 0, n_max = 0;
    size_t off = layout(1, &grid, &n_max);
    bool aligned = force_aligned || (nrb >= grid_max && (double)nrb / ((double)per_cta_rb * grid_max) >= 0.8);
    if (!aligned && chunks_of(n_max) <= kMaxSlots && off + (size_t)chunks_of(n_max) * kSlotBytes <= kCoResidentBytes)
        aligned = true;
    if (!aligned) off = layout(0, &grid, &n_max);
    // Long rows, one FP16 vector: the staged activations (4 bytes per column) crowd out the ring
    // and every CTA converts the whole vector.  Clusters of two CTAs then share whole row
    // blocks and each CTA takes one half of the columns: half the staging time and footprint, a
    // deeper ring, and the halves' sums meet in the first CTA's shared memory.  Needs runs of
    // whole chunks (groups a multiple of 8) and at least 8 tiles per warp in every CTA, so that
    // warp ranges start on chunk boundaries and no chunk straddles a run.
    if (TLLM_GEMV_KSPLIT && allow_clusters && aligned && mode == kF16 && nvt == 1 && a.batch == 1 &&
        cols >= TLLM_GEMV_KSPLIT_MIN_COLS && (a.groups % (2 * kSlotTiles)) == 0 && grid_max >= 2) {
        const int parts = nrb < grid_max / 2 ? nrb : grid_max / 2;
        if ((nrb / parts) * (a.groups / 2) >= 8 * kWarps) off = layout(2, &grid, &n_max);
    }
    a.late_release = release_rule(rows, cols);
    // Ring: what a CTA can use, bounded by what lets two CTAs share the SM (the launch that
    // follows prefetches its weights beside this one); a problem whose activations leave less
    // than kMinSharedSlots slots that way runs one CTA per SM with all of the shared memory.
    const int want = chunks_of(n_max) > kMaxSlots ? kMaxSlots : chunks_of(n_max);
    long long slots = ((long long)kCoResidentBytes - (long long)off) / kSlotBytes;
    if (slots < kWarps || (slots < want && slots < kMinSharedSlots)) slots = ((long long)kMaxSmemBytes - (long long)off) / kSlotBytes;
    if (slots > want) slots = want;
    if (slots < kWarps)
        return fail(TLLM_ERR_SIZE, "rows=%d cols=%d with %d vectors per pass needs more shared memory than an SM has "
                    "(%zu bytes before the ring)", rows, cols, nvt, off);
    a.ring_slots = (int)slots;
    // Staging shared by pairs of CTAs (clusters of two; each converts half of the activations and
    // writes into both shared memories): for passes of three and four vectors, where every thread
    // converts several 8-element items (measured: 14336x4096 at four vectors 9.2 -> 8.3 us,
    // 4096x14336 16.4 -> 13.7 us).  One vector of a long row gains nothing: 4096x14336 9.4 us
    // either way, the stores into the partner's shared memory and the two cluster barriers cost
    // what the halved conversion saves.
    a.pair = (TLLM_GEMV_PAIR_STAGING && allow_clusters && !i8 && !a.ksplit && !a.x_local && (grid % 2) == 0 && a.batch >= 3 &&
              (long long)a.groups * 16 * a.batch >= 2 * kThreads) ? 1 : 0;
    // only where the ring is shallow (fewer than two slots per warp): a deeper ring hides the HBM
    // latency by itself and the prefetch instructions then only cost issue slots
    a.l2_prefetch = (chunks_of(n_max) > (int)slots && slots < 2 * kWarps) ? 1 : 0;
    off += (size_t)slots * kSlotBytes;
    *grid_out = grid;
    *smem_out = off;
    return TLLM_OK;
}

template <int MODE, int NB, int NV, bool AR = false, bool KS = false>
static int launch_mode(const GemvArgs& a, int grid, size_t smem, cudaStream_t stream)
{
    static bool attr[64] = {};
    static std::mutex mu;
    int dev = 0;
    cudaGetDevice(&dev);
    {
        std::lock_guard<std::mutex> lk(mu);
        if (dev >= 0 && dev < 64 && !attr[dev]) {
            const cudaError_t e1 = cudaFuncSetAttribute(gemv_packed_kernel<MODE, NB, NV, AR, KS>,
                                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxSmemBytes);
            const cudaError_t e2 = cudaFuncSetAttribute(gemv_packed_kernel<MODE, NB, NV, AR, KS>,
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
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (a.pair || a.ksplit) {       // clusters of two CTAs (plan_gemv made the grid even)
        at[1].id = cudaLaunchAttributeClusterDimension;
        at[1].val.clusterDim.x = 2;
        at[1].val.clusterDim.y = 1;
        at[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_packed_kernel<MODE, NB, NV, AR, KS>, a);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(TLLM_ERR_LAUNCH, "gemv_packed launch: %s", cudaGetErrorString(e));
    }
    return TLLM_OK;
}

// Vectors per pass as instantiated for a batch of 1..4 FP16 vectors.
static inline int f16_nvt(int batch) { return batch <= 1 ? 1 : (batch == 2 ? 2 : 4); }
// FP16 vectors: one or two ride the 24-bit digits, three and four the wide 16-bit mode
static inline int f16_mode(int mode, int batch) { return (mode == kF16 && batch >= 3) ? kF16W : mode; }

static int dispatch(const GemvArgs& a, int mode, int grid, size_t smem, cudaStream_t stream)
{
    switch (mode) {
        case kF16:
            if (a.batch <= 1 && a.ksplit) return launch_mode<kF16, 1, 1, false, true>(a, grid, smem, stream);
            if (a.batch <= 1) return launch_mode<kF16, 1, 1>(a, grid, smem, stream);
            return launch_mode<kF16, 1, 2>(a, grid, smem, stream);
        case kF16W: return launch_mode<kF16W, 1, 4>(a, grid, smem, stream);
        case kF16Norm: return launch_mode<kF16Norm, 1, 1>(a, grid, smem, stream);
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
    mode = f16_mode(mode, batch);
    if ((st = plan_gemv(a, s->sms, mode, (mode == kF16 || mode == kF16W) ? f16_nvt(batch) : 1, kMaxCtas, false, &grid, &smem,
                        mode != kF16Norm)))
        return st;
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
// packed back to back (every row count but the last a multiple of 16) are one contiguous
// tile array and are streamed as ONE matrix in one launch, outputs scattered per
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
                contiguous = contiguous && (rows[i] % kTileRows == 0) && (packed[i + 1] == packed[i] + packed_bytes(rows[i], cols));
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

// FP16 GEMV over 1..4 matrices packed back to back whose shared input vector is made in the
// kernel's staging phase: x = rmsnorm(a (+ b)) * w, the rounded sum a + b stored to res_out.
int launch_gemv_packed_multi_norm(int count, const uint8_t* const* packed, half* const* y, const int* rows, int cols,
                                  const half* a, const half* b, const half* w, half* res_out, float eps,
                                  cudaStream_t stream)
{
    const FusedX fx = {a, b, w, res_out, eps};
    if (count == 1)
        return launch_packed_once(packed[0], nullptr, y[0], 1.0f, kF16Norm, 1, rows[0], cols, stream, nullptr, &fx);
    SegY seg = {};
    seg.n = count;
    int total = 0;
    for (int i = 0; i < count; i++) {
        if (i + 1 < count && ((rows[i] % kTileRows) != 0 || packed[i + 1] != packed[i] + packed_bytes(rows[i], cols)))
            return fail(TLLM_ERR_SHAPE, "gemv_packed_multi_norm: the matrices must be packed back to back "
                        "(row counts multiples of %d but the last)", kTileRows);
        seg.rows[i] = rows[i];
        seg.y[i] = y[i];
        total += rows[i];
    }
    return launch_packed_once(packed[0], nullptr, nullptr, 1.0f, kF16Norm, 1, total, cols, stream, nullptr, &fx, &seg);
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
// loads the library carries these 40 KB until the process exits.
//   [0, 40960)        partial-sum records, kNoAllocMaxCtas x 2 x 16 words {value, flag} (one vector)
//   [40960, 40964)    device error flag
constexpr int kNoAllocMaxRows = 65536;
constexpr int kNoAllocMaxCtas = 160;
constexpr size_t kNoAllocWsBytes = (size_t)kNoAllocMaxCtas * 2 * kTileRows * sizeof(uint2);
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
// (different streams) race.  With one vector a partial record is 16 words, so the records
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
    a.ws_stride = 2 * kTileRows;
    // the records' flags must start at zero; a call that was cut short may have left some set
    if (cudaMemsetAsync(a.ws, 0, (size_t)grid * 2 * kTileRows * sizeof(uint2), stream) != cudaSuccess) {
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
    if ((st = plan_gemv(a, s->sms, kF16, 1, kMaxCtas, true, &grid, &smem, true))) return st;
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
    if (a.ksplit) return launch_mode<kF16, 1, 1, true, true>(a, grid, smem, stream);
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
    const long long threads = (long long)((rows + kTileRows - 1) / kTileRows) * (cols / kGroup) * 128;
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
