// Prefill GEMM  C[M,N] = A[M,K] . W^T  on the 5th-generation tensor cores (sm_100a).
//
// W is ternary with one FP16 scale per 128 weights along K.  The product
// scale * t is exactly representable in FP16, so the weight operand is expanded to
// FP16 {-s, 0, +s} and a plain FP16 x FP16 -> FP32 contraction over the whole K
// gives the reference result with nothing but FP32 accumulation rounding.
//
// One CTA computes a tile of 128 output features x 256 tokens:
//   * the weight tile is the MMA's A operand and lives in TENSOR MEMORY: four
//     expander warps (one thread per feature row = one TMEM lane) read the row's
//     packed 2-bit codes (packed_layout.cuh) straight from global/L2 and expand 128
//     weights per stage: the codes c = t + 1 of two weights become the selector of one
//     PRMT into the byte table {-s, 0, +s} of the group's scale (an integer multiply-add
//     builds the selector), which yields the FP16 pair directly; tcgen05.st writes
//     them.  The expanded weights never touch shared memory, which leaves its
//     bandwidth to the activation operand;
//   * the activation tile [256 tokens x 128 K] is the B operand in shared memory,
//     brought by TMA (two 128-byte-swizzled boxes of 64 K per stage, 3 stages);
//   * one thread issues tcgen05.mma (kind::f16, M=128, N=256, K=16; A from TMEM, B
//     from a shared-memory descriptor) into a 128 x 256 FP32 accumulator in TMEM;
//   * the expander warps then read the accumulator back with tcgen05.ld and store
//     C (a TMEM lane is an output feature, so a warp writes 32 adjacent features
//     of one token at a time).
// TMEM: columns 0..255 accumulator, 256..383 two weight stages of 64 columns.
// All mbarrier waits are bounded; a wait that gives up sets the device error flag
// and every role falls through to the common exit, where TMEM is released.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "packed_layout.cuh"

namespace tllm {

namespace gemm {

constexpr int kTileN = 128;          // output features per CTA (MMA M, TMEM lanes)
constexpr int kStageK = 128;         // K per pipeline stage = one scale group
constexpr int kAStages = 2;          // weight stages in tensor memory
constexpr int kBoxK = 64;            // TMA box inner extent (128 bytes of FP16)
constexpr int kThreads = 256;
constexpr int kAColsPerStage = kStageK / 2;            // 64 columns of FP16 pairs

// Per token-tile size TM (tokens per CTA = MMA N): 256 for long prefills; 128/64/32 for
// short ones and for decode batches, where two CTAs share an SM (half the shared memory
// and half the tensor memory each) so that twice as many warps expand weights.
template <int TM>
struct Cfg {
    static constexpr int kBoxBytes = TM * kBoxK * 2;
    static constexpr int kStageBytes = 2 * kBoxBytes;                    // TM x 128 K x FP16
    static constexpr int kBStages = (TM == 256) ? 3 : (TM == 128) ? 3 : (TM == 64) ? 6 : 8;
    static constexpr int kAccCols = TM;                                  // FP32 accumulator columns
    static constexpr int kTmemCols = (TM == 256) ? 512 : 256;            // power of two >= TM + 128
    static constexpr int kCtasPerSm = (TM == 256) ? 1 : 2;
    static constexpr size_t kSmem = (size_t)kBStages * kStageBytes + 1024;
};

struct Args {
    const uint8_t* packed;     // packed weights [ceil(N/16)][K/128] tiles
    half* C;                   // [M, N]
    int M, N, K, groups;       // groups = K / 128
    int nrb;                   // ceil(N / 16)
    int* err;
    // split-K (gridDim.z > 1): CTA z contracts stages [z*groups/ks, (z+1)*groups/ks) and writes an
    // FP32 partial tile; the CTA of a tile that arrives last adds the partials in z order.
    float* ws;                 // [tile][z][tokens of the tile][128] FP32
    unsigned* counters;        // [tiles], zero between launches
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

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128
// bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_b_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);          // start address
    d |= (uint64_t)1 << 16;                                 // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                       // stride byte offset: 8 rows x 128 B
    d |= (uint64_t)1 << 46;                                 // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                                 // layout: 128-byte swizzle
    return d;
}

// kind::f16 instruction descriptor: FP16 x FP16 -> FP32, both operands K-major.
template <int TM>
__device__ __forceinline__ uint32_t make_idesc()
{
    uint32_t d = 0;
    d |= 1u << 4;                          // D format F32
    d |= 0u << 7;                          // A format F16
    d |= 0u << 10;                         // B format F16
    d |= (uint32_t)(TM >> 3) << 17;        // N
    d |= (uint32_t)(kTileN >> 4) << 24;    // M
    return d;
}

__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
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
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}

template <int TM>
__global__ void __launch_bounds__(kThreads, Cfg<TM>::kCtasPerSm)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const Args a)
{
    constexpr int kBStages = Cfg<TM>::kBStages, kStageBytes = Cfg<TM>::kStageBytes, kBoxBytes = Cfg<TM>::kBoxBytes;
    constexpr int kAccCols = Cfg<TM>::kAccCols, kTmemCols = Cfg<TM>::kTmemCols, kTileM = TM;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the 128-byte swizzle atoms
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bars[2 * kBStages + 2 * kAStages + 1];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ int last_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * kTileN;          // first output feature of the tile
    const int m0 = blockIdx.y * kTileM;          // first token of the tile
    const int ks = gridDim.z;
    const int it0 = (int)(((long long)blockIdx.z * a.groups) / ks);          // first scale group of this CTA
    const int nstages = (int)(((long long)(blockIdx.z + 1) * a.groups) / ks) - it0;   // one scale group per stage

    const uint32_t bar0 = smem_u32(bars);
    auto full_b = [&](int s) { return bar0 + 8u * s; };
    auto empty_b = [&](int s) { return bar0 + 8u * (kBStages + s); };
    auto full_a = [&](int s) { return bar0 + 8u * (2 * kBStages + s); };
    auto empty_a = [&](int s) { return bar0 + 8u * (2 * kBStages + kAStages + s); };
    const uint32_t acc_full = bar0 + 8u * (2 * kBStages + 2 * kAStages);

    if (tid == 0) {
        for (int s = 0; s < kBStages; s++) {
            mbar_init(full_b(s), 1);
            mbar_init(empty_b(s), 1);
        }
        for (int s = 0; s < kAStages; s++) {
            mbar_init(full_a(s), 128);
            mbar_init(empty_a(s), 1);
        }
        mbar_init(acc_full, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {       // one warp allocates all 512 TMEM columns of this SM
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_slot;
    volatile int* abortp = &abort_flag;

    if (warp == 0) {
        // ---------------- TMA producer: activations ----------------
        if (lane == 0) {
            for (int it = 0; it < nstages; it++) {
                const int s = it % kBStages;
                if (!mbar_wait(empty_b(s), ((it / kBStages) & 1) ^ 1, abortp)) { abort_flag = 1; break; }
                mbar_expect_tx(full_b(s), kStageBytes);
                const uint32_t dst = smem_u32(smem + (size_t)s * kStageBytes);
                tma_load_2d(dst, &map_a, (it0 + it) * kStageK, m0, full_b(s));
                tma_load_2d(dst + kBoxBytes, &map_a, (it0 + it) * kStageK + kBoxK, m0, full_b(s));
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc<TM>();
            for (int it = 0; it < nstages; it++) {
                const int sb = it % kBStages, sa = it % kAStages;
                if (!mbar_wait(full_b(sb), (it / kBStages) & 1, abortp) ||
                    !mbar_wait(full_a(sa), (it / kAStages) & 1, abortp)) { abort_flag = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t bsm = smem_u32(smem + (size_t)sb * kStageBytes);
                const uint32_t a_t = tmem + kAccCols + sa * kAColsPerStage;
#pragma unroll
                for (int k = 0; k < kStageK / 16; k++) {
                    // K step of 16: 32 bytes inside the 128-byte swizzled row; second box after 64 K
                    const uint64_t bd = make_b_desc(bsm + (k >> 2) * kBoxBytes + (k & 3) * 32);
                    mma_ts(tmem, a_t + k * 8, bd, idesc, (it > 0 || k > 0) ? 1u : 0u);
                }
                mma_commit(empty_b(sb));
                mma_commit(empty_a(sa));
            }
            mma_commit(acc_full);
        }
    } else if (warp >= 4) {
        // ---------------- weight expanders, then epilogue ----------------
        const int row = tid - 128;                       // feature row inside the tile = TMEM lane
        const int n = n0 + row;
        const int rb = n >> 4, r16 = n & 15;             // 16-row block and row inside it
        const int gq = r16 & 7, h = r16 >> 3;
        const bool row_valid = rb < a.nrb;               // rows past the matrix expand to zeros
        const uint8_t* tile0 = a.packed + ((size_t)(row_valid ? rb : 0) * a.groups + it0) * kTileBytes;
        // this row's code words of MMA lane t: the pair (column halves j2 = 0, 1) at word index
        // (gq*4 + t)*4 + 2h, i.e. one 64-bit load per t; each word holds all four 32-column steps
        const int pair0 = (gq * 4) * 2 + h;              // in units of uint2; + t*2
        const int spos = tile_scale_index(r16);
        const uint32_t lane_base = tmem + ((uint32_t)(row & ~31) << 16);   // this warp's 32 TMEM lanes

        uint2 cw[4];
        uint32_t sbits = 0;
        auto load_stage = [&](const uint8_t* tp) {
            const uint2* p = reinterpret_cast<const uint2*>(tp) + pair0;
#pragma unroll
            for (int t = 0; t < 4; t++) cw[t] = __ldg(p + t * 2);
            sbits = __half_as_ushort(__ldg(reinterpret_cast<const half*>(tp + kTileCodeBytes) + spos));
        };
        if (row_valid) load_stage(tile0);
        bool ok = true;
        for (int it = 0; it < nstages; it++) {
            const int sa = it % kAStages;
            // PRMT table of this stage: bytes 0,1 = -s (code 0), 2,3 = 0 (code 1), 4,5 = +s (code 2)
            const uint32_t tab_lo = row_valid ? (sbits ^ 0x8000u) : 0u, tab_hi = row_valid ? sbits : 0u;
            uint2 cur[4];
#pragma unroll
            for (int t = 0; t < 4; t++) cur[t] = cw[t];
            if (it + 1 < nstages && row_valid) load_stage(tile0 + (size_t)(it + 1) * kTileBytes);   // prefetch the next group
            if (!mbar_wait(empty_a(sa), ((it / kAStages) & 1) ^ 1, abortp)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_t = lane_base + kAccCols + sa * kAColsPerStage;
#pragma unroll
            for (int m = 0; m < 4; m++) {                 // 32 K per step -> 16 columns; step m is code field m
                uint32_t r[16];
#pragma unroll
                for (int t = 0; t < 4; t++) {
#pragma unroll
                    for (int j2 = 0; j2 < 2; j2++) {
                        // four codes (K offsets 32m + 16*j2 + 4t .. +3) in the low two bits of each byte
                        const uint32_t y = ((j2 ? cur[t].y : cur[t].x) >> (2 * m)) & 0x03030303u;
                        // selector nibbles 2c, 2c+1 per weight: one PRMT makes an FP16 pair {-s,0,+s}
                        r[8 * j2 + 2 * t] = prmt(tab_lo, tab_hi, y * 0x22u + 0x1010u);
                        r[8 * j2 + 2 * t + 1] = prmt(tab_lo, tab_hi, (y >> 16) * 0x22u + 0x1010u);
                    }
                }
                tmem_st16(a_t + m * 16, r);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(full_a(sa));
        }
        if (!ok) abort_flag = 1;

        // ---------------- epilogue: accumulator -> C ----------------
        const bool good = ok && mbar_wait(acc_full, 0, abortp);
        const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
        if (good) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float* wtile = a.ws + ((size_t)tile_id * ks + blockIdx.z) * kTileM * kTileN;
#pragma unroll 1
            for (int cchunk = 0; cchunk < kTileM / 32; cchunk++) {
                if (m0 + cchunk * 32 >= a.M) break;       // uniform: no tokens left in this chunk
                uint32_t v[32];
                tmem_ld32(lane_base + cchunk * 32, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (ks == 1) {
                    if (n < a.N) {
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const int m = m0 + cchunk * 32 + j;
                            if (m < a.M) a.C[(size_t)m * a.N + n] = __float2half_rn(__uint_as_float(v[j]));
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (m0 + cchunk * 32 + j < a.M) wtile[(size_t)(cchunk * 32 + j) * kTileN + row] = __uint_as_float(v[j]);
                }
            }
        } else {
            abort_flag = 1;
        }
        if (ks > 1) {
            // publish, count, and let the last CTA of the tile add the partials in z order (all 128
            // epilogue threads take part in the two barriers whether or not their wait succeeded)
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (row == 0) {
                const unsigned prev = atomicAdd(a.counters + tile_id, 1u);
                last_flag = (prev == (unsigned)ks - 1u) ? 1 : 0;
                if (last_flag) a.counters[tile_id] = 0;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (ks > 1 && last_flag && !abort_flag) {
        // The tile's last CTA adds the partial tiles in z order, all eight warps: lane l sums
        // features 4l..4l+3 (one 16-byte load per partial), warps take tokens round-robin, eight
        // tokens per trip so that 8 * ks loads are in flight per thread.
        __threadfence();
        const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
        const int f4 = lane * 4;
        const float* base = a.ws + (size_t)tile_id * ks * kTileM * kTileN + f4;
        const int mt = min(kTileM, a.M - m0);
        for (int mb = warp * 8; mb < mt; mb += 8 * (kThreads / 32)) {
            float4 tot[8];
#pragma unroll
            for (int u = 0; u < 8; u++) tot[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int z = 0; z < ks; z++) {
                float4 p[8];
#pragma unroll
                for (int u = 0; u < 8; u++)
                    p[u] = (mb + u < mt) ? __ldcg(reinterpret_cast<const float4*>(base + ((size_t)z * kTileM + mb + u) * kTileN))
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    tot[u].x += p[u].x;
                    tot[u].y += p[u].y;
                    tot[u].z += p[u].z;
                    tot[u].w += p[u].w;
                }
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                if (mb + u >= mt) continue;
                half* cp = a.C + (size_t)(m0 + mb + u) * a.N + n0 + f4;
                const float v[4] = {tot[u].x, tot[u].y, tot[u].z, tot[u].w};
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (n0 + f4 + j < a.N) cp[j] = __float2half_rn(v[j]);
            }
        }
    }
    if (abort_flag && tid == 0) atomicExch(a.err, TLLM_ERR_TIMEOUT);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point query, so that the
// library has no link-time dependency on libcuda (it must load on machines without a driver).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

}  // namespace gemm


bool gemm_tcgen05_supported(int M, int N, int K)
{
    (void)N;
    return M >= 1 && K >= gemm::kStageK && K % gemm::kStageK == 0;
}

// Scratch of the split-K path: 4 regions handed out round-robin, so that launches on up to four
// streams do not share one (launches on one stream are ordered).
namespace gemm {
constexpr size_t kSplitWsBytes = (size_t)24 << 20;
constexpr int kSplitTickets = 4;
constexpr int kSplitMaxTiles = 4096;
struct SplitScratch {
    float* ws = nullptr;
    unsigned* counters = nullptr;
    int sms = 0;
    unsigned ticket = 0;
    bool ready = false, failed = false;
};
static SplitScratch g_split[64];
static std::mutex g_split_mu;
}  // namespace gemm

template <int TM>
static int launch_tm(gemm::EncodeTiledFn enc, const half* A, const gemm::Args& a_in, cudaStream_t stream)
{
    using namespace gemm;
    Args a = a_in;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)a.K, (cuuint64_t)a.M};
    const cuuint64_t strides[1] = {(cuuint64_t)a.K * sizeof(half)};
    const cuuint32_t box[2] = {(cuuint32_t)kBoxK, (cuuint32_t)TM};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<half*>(A), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TLLM_ERR_LAUNCH, "cuTensorMapEncodeTiled failed with %d", (int)r);
    static bool attr[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr[dev]) {
        cudaFuncSetAttribute(gemm_kernel<TM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<TM>::kSmem);
        cudaFuncSetAttribute(gemm_kernel<TM>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        attr[dev] = true;
    }
    dim3 grid((a.N + kTileN - 1) / kTileN, (a.M + TM - 1) / TM, 1);
    // Too few tiles for the SMs: split K (at most four ways).
    if (dev >= 0 && dev < 64) {
        std::lock_guard<std::mutex> lk(g_split_mu);
        SplitScratch& sc = g_split[dev];
        if (!sc.sms) cudaDeviceGetAttribute(&sc.sms, cudaDevAttrMultiProcessorCount, dev);
        const int tiles = (int)(grid.x * grid.y), slots = sc.sms * Cfg<TM>::kCtasPerSm;
        int ks = 1;
        if (tiles * 2 <= slots) ks = slots / tiles;
        if (ks > a.groups / 8) ks = a.groups / 8;        // at least eight scale groups per split
        if (ks > 4) ks = 4;
        if (ks > 1 && tiles <= kSplitMaxTiles && (size_t)tiles * ks * TM * kTileN * sizeof(float) <= kSplitWsBytes && !sc.failed) {
            if (!sc.ready) {
                if (cudaMalloc(&sc.ws, kSplitWsBytes * kSplitTickets) != cudaSuccess ||
                    cudaMalloc(&sc.counters, sizeof(unsigned) * kSplitMaxTiles * kSplitTickets) != cudaSuccess) {
                    cudaGetLastError();
                    sc.failed = true;
                } else {
                    cudaMemset(sc.counters, 0, sizeof(unsigned) * kSplitMaxTiles * kSplitTickets);
                    sc.ready = true;
                }
            }
            if (sc.ready) {
                const unsigned t = sc.ticket++ % kSplitTickets;
                a.ws = sc.ws + (size_t)t * (kSplitWsBytes / sizeof(float));
                a.counters = sc.counters + (size_t)t * kSplitMaxTiles;
                grid.z = ks;
            }
        }
    }
    gemm_kernel<TM><<<grid, kThreads, Cfg<TM>::kSmem, stream>>>(map, a);
    return check_launch("gemm_tcgen05");
}

// A: half [M,K] row-major (16-byte aligned), packed: prepared weights of [N,K], C: half [M,N].
int launch_gemm_tcgen05(const half* A, const uint8_t* packed, half* C, int M, int N, int K, cudaStream_t stream)
{
    using namespace gemm;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return fail(TLLM_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from this driver");
    int* err = device_error_flag();
    if (!err) return fail(TLLM_ERR_LAUNCH, "device scratch unavailable");
    Args a;
    a.packed = packed;
    a.C = C;
    a.M = M;
    a.N = N;
    a.K = K;
    a.groups = K / kStageK;
    a.nrb = (N + kTileRows - 1) / kTileRows;
    a.err = err;
    a.ws = nullptr;
    a.counters = nullptr;
    // token tile: the smallest that holds M, 256 for long prefills
    if (M <= 32) return launch_tm<32>(enc, A, a, stream);
    if (M <= 64) return launch_tm<64>(enc, A, a, stream);
    if (M <= 128) return launch_tm<128>(enc, A, a, stream);
    return launch_tm<256>(enc, A, a, stream);
}

}  // namespace tllm
