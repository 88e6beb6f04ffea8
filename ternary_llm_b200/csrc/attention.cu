// Causal attention over the FP16 KV cache with grouped-query heads.
//
// Semantics of the reference operator (include/kernels.cuh:55-58, kernels/attention.cu):
//   q, output: [batch, seq_len, n_heads, head_dim];  caches: [batch, n_kv_heads,
//   kv_len_max, head_dim];  query s of a call with seq_len tokens sits at position
//   kv_len - seq_len + s and attends to cache positions 0..that position;
//   scores = q.k / sqrt(head_dim), softmax in FP32, output = P.V rounded to FP16.
// (The reference's multi-token kernel normalises by a per-thread partial sum,
// kernels/attention.cu:230-296, which does not compute a softmax; this implementation
// computes the softmax that its header comment describes for every seq_len.)
//
// One CTA serves one KV head and ALL the query heads that share it, so K and V are read
// once per group instead of once per query head.  The CTA walks its range of cache
// positions in chunks of 256 with an online softmax.  A chunk of K and of V is one
// contiguous block of the cache ([position][head_dim]); each is brought into shared
// memory by a single bulk copy (cp.async.bulk, completion on an mbarrier, bounded wait),
// so the whole chunk is in flight at once instead of one dependent load per position:
//   scores  - one thread per position, dot products against the group's query heads
//             (queries pre-scaled in shared memory); the 16-byte pieces of a row are
//             visited in an order rotated by the position, which keeps the eight lanes
//             of a shared-memory phase on different banks;
//   softmax - one warp per query head over the chunk's 256 scores;
//   P.V     - one thread per (query head, channel), V rows read from shared memory.
// Decode (seq_len == 1) splits the cache positions over several CTAs (one chunk each);
// each writes (max, sum, unnormalised output) and the CTA that arrives last on a counter
// merges them in split order and resets the counter, so replays of a captured graph need
// no host-side clearing.  The cache length can come from device memory for that case.
#include <cfloat>

#include "launch.cuh"
#include "layer.cuh"

namespace tllm {

constexpr int kAttnThreads = 256;
constexpr int kAttnChunk = 256;       // cache positions per pass = per decode split
constexpr int kAttnMaxGroup = 16;     // query heads per KV head
constexpr int kAttnMaxElems = 16;     // outputs per thread: group * head_dim / 256

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Bounded wait on an mbarrier phase (about a second at most); false = gave up.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity)
{
#pragma unroll 1
    for (int i = 0; i < (1 << 22); i++) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

struct AttnArgs {
    const half* q;
    const half* k_cache;
    const half* v_cache;
    half* out;
    int n_heads, n_kv_heads, head_dim, seq_len, kv_len, kv_len_max;
    const int* kv_len_dev;     // decode: kv_len = *kv_len_dev + kv_len when not null
    int nsplit;                // decode: CTAs per (batch, kv head); 1 otherwise
    float* ws;                 // [batch * n_kv_heads][nsplit][group * (head_dim + 2)]
    unsigned* counters;        // [batch * n_kv_heads]
    int* err;                  // device error flag (set when a bounded wait gives up)
};

__global__ void __launch_bounds__(kAttnThreads)
attention_kernel(const AttnArgs a)
{
    extern __shared__ __align__(16) float smem[];
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hd = a.head_dim;
    const int G = a.n_heads / a.n_kv_heads;
    const int kvh = blockIdx.y, b = blockIdx.z;
    const bool decode = (a.seq_len == 1);
    const int s_idx = decode ? 0 : blockIdx.x;
    const int split = decode ? blockIdx.x : 0;

    half* ks = reinterpret_cast<half*>(smem);                 // [kAttnChunk][hd] K chunk
    half* vs = ks + kAttnChunk * hd;                          // [kAttnChunk][hd] V chunk
    float* qs = reinterpret_cast<float*>(vs + kAttnChunk * hd);   // [G][hd] queries times 1/sqrt(hd)
    float* ps = qs + G * hd;                  // [G][kAttnChunk] scores, then probabilities
    float* m_run = ps + G * kAttnChunk;       // [G] running maximum
    float* l_run = m_run + kAttnMaxGroup;     // [G] running sum
    float* corr = l_run + kAttnMaxGroup;      // [G] rescale factor of this chunk
    __shared__ int s_last;
    __shared__ int s_ok;
    __shared__ __align__(8) unsigned long long s_bar;
    const uint32_t bar = smem_u32(&s_bar);
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }

    pdl_wait();
    int kv_len = a.kv_len;
    if (a.kv_len_dev) kv_len += *a.kv_len_dev;
    const int limit = kv_len - a.seq_len + s_idx + 1;          // positions [0, limit) are visible
    int lo = 0, hi = limit, nactive = 1;
    if (decode) {
        nactive = (limit + kAttnChunk - 1) / kAttnChunk;
        if (nactive > a.nsplit) nactive = a.nsplit;            // the last split takes the rest
        if (split >= nactive) return;
        lo = split * kAttnChunk;
        hi = (split == nactive - 1) ? limit : lo + kAttnChunk;
    }

    const float scale = rsqrtf((float)hd);
    const half* qp = a.q + (((size_t)b * a.seq_len + s_idx) * a.n_heads + (size_t)kvh * G) * hd;
    for (int i = tid; i < G * hd; i += kAttnThreads) qs[i] = __half2float(qp[i]) * scale;
    if (tid < G) {
        m_run[tid] = -FLT_MAX;
        l_run[tid] = 0.f;
    }
    const size_t cache_base = ((size_t)b * a.n_kv_heads + kvh) * (size_t)a.kv_len_max * hd;
    const half* kb = a.k_cache + cache_base;
    const half* vb = a.v_cache + cache_base;

    const int nelem = (G * hd + kAttnThreads - 1) / kAttnThreads;
    float o[kAttnMaxElems];
#pragma unroll
    for (int e = 0; e < kAttnMaxElems; e++) o[e] = 0.f;
    __syncthreads();

    uint32_t phase = 0;
    for (int c0 = lo; c0 < hi; c0 += kAttnChunk) {
        const int nc = min(kAttnChunk, hi - c0);
        // ---- stage the chunk: one bulk copy each for K and V -----------------------
        if (tid == 0) {
            const uint32_t bytes = (uint32_t)nc * hd * sizeof(half);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(2 * bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(ks)), "l"(kb + (size_t)c0 * hd), "r"(bytes), "r"(bar) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(vs)), "l"(vb + (size_t)c0 * hd), "r"(bytes), "r"(bar) : "memory");
            s_ok = mbar_wait_bounded(bar, phase) ? 1 : 0;
        }
        phase ^= 1u;
        __syncthreads();
        if (!s_ok) {                       // uniform: the copy never completed
            if (tid == 0 && a.err) atomicExch(a.err, TLLM_ERR_TIMEOUT);
            return;
        }
        // ---- scores: thread j <-> position c0 + j --------------------------------
        if (tid < nc) {
            float dot[kAttnMaxGroup];
#pragma unroll
            for (int g = 0; g < kAttnMaxGroup; g++) dot[g] = 0.f;
            const uint4* k4 = reinterpret_cast<const uint4*>(ks + (size_t)tid * hd);
            const int nd8 = hd >> 3;
            for (int i8 = 0; i8 < nd8; i8++) {
                int d8 = i8 + tid;
                d8 -= (d8 / nd8) * nd8;                    // (i8 + tid) % nd8
                const uint4 raw = k4[d8];
                const half2* h = reinterpret_cast<const half2*>(&raw);
                float kf[8];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 f = __half22float2(h[j]);
                    kf[2 * j] = f.x;
                    kf[2 * j + 1] = f.y;
                }
#pragma unroll
                for (int g = 0; g < kAttnMaxGroup; g++) {
                    if (g < G) {
                        const float4 q0 = *reinterpret_cast<const float4*>(qs + g * hd + d8 * 8);
                        const float4 q1 = *reinterpret_cast<const float4*>(qs + g * hd + d8 * 8 + 4);
                        dot[g] += kf[0] * q0.x + kf[1] * q0.y + kf[2] * q0.z + kf[3] * q0.w + kf[4] * q1.x +
                                  kf[5] * q1.y + kf[6] * q1.z + kf[7] * q1.w;
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < kAttnMaxGroup; g++)
                if (g < G) ps[g * kAttnChunk + tid] = dot[g];
        }
        __syncthreads();
        // ---- online softmax: warp w <-> heads w, w + 8 ----------------------------
        for (int g = warp; g < G; g += kAttnThreads / 32) {
            float* p = ps + g * kAttnChunk;
            float mx = -FLT_MAX;
            for (int j = lane; j < nc; j += 32) mx = fmaxf(mx, p[j]);
            mx = warp_max(mx);
            const float m_old = m_run[g];
            const float m_new = fmaxf(m_old, mx);
            float sum = 0.f;
            for (int j = lane; j < nc; j += 32) {
                const float e = __expf(p[j] - m_new);
                p[j] = e;
                sum += e;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float c = __expf(m_old - m_new);       // 0 for the first chunk (m_old = -FLT_MAX)
                corr[g] = c;
                l_run[g] = l_run[g] * c + sum;
                m_run[g] = m_new;
            }
        }
        __syncthreads();
        // ---- P.V: thread <-> (head g, channel d) ----------------------------------
#pragma unroll
        for (int e = 0; e < kAttnMaxElems; e++) {
            if (e < nelem) {
                const int idx = e * kAttnThreads + tid;
                if (idx < G * hd) {
                    const int g = idx / hd, d = idx - g * hd;
                    const float* p = ps + g * kAttnChunk;
                    const half* vp = vs + d;
                    float acc0 = o[e] * corr[g], acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
                    int j = 0;
                    for (; j + 4 <= nc; j += 4) {
                        acc0 = fmaf(p[j], __half2float(vp[(j + 0) * hd]), acc0);
                        acc1 = fmaf(p[j + 1], __half2float(vp[(j + 1) * hd]), acc1);
                        acc2 = fmaf(p[j + 2], __half2float(vp[(j + 2) * hd]), acc2);
                        acc3 = fmaf(p[j + 3], __half2float(vp[(j + 3) * hd]), acc3);
                    }
                    for (; j < nc; j++) acc0 = fmaf(p[j], __half2float(vp[j * hd]), acc0);
                    o[e] = (acc0 + acc1) + (acc2 + acc3);
                }
            }
        }
        __syncthreads();
    }

    half* op = a.out + (((size_t)b * a.seq_len + s_idx) * a.n_heads + (size_t)kvh * G) * hd;
    if (!decode || nactive == 1) {
#pragma unroll
        for (int e = 0; e < kAttnMaxElems; e++) {
            if (e < nelem) {
                const int idx = e * kAttnThreads + tid;
                if (idx < G * hd) {
                    const float l = l_run[idx / hd];
                    op[idx] = __float2half_rn(l > 0.f ? o[e] / l : 0.f);
                }
            }
        }
        return;
    }

    // ---- decode with several splits: publish, last arriver merges ------------------
    const int rec = G * (hd + 2);
    float* my = a.ws + ((size_t)(b * a.n_kv_heads + kvh) * a.nsplit + split) * rec;
#pragma unroll
    for (int e = 0; e < kAttnMaxElems; e++) {
        if (e < nelem) {
            const int idx = e * kAttnThreads + tid;
            if (idx < G * hd) my[idx] = o[e];
        }
    }
    if (tid < G) {
        my[G * hd + tid] = m_run[tid];
        my[G * hd + G + tid] = l_run[tid];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned* cnt = a.counters + b * a.n_kv_heads + kvh;
        s_last = (atomicAdd(cnt, 1u) == (unsigned)(nactive - 1)) ? 1 : 0;
        if (s_last) *cnt = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float* base = a.ws + (size_t)(b * a.n_kv_heads + kvh) * a.nsplit * rec;
#pragma unroll
    for (int e = 0; e < kAttnMaxElems; e++) {
        if (e < nelem) {
            const int idx = e * kAttnThreads + tid;
            if (idx < G * hd) {
                const int g = idx / hd;
                float m = -FLT_MAX;
                for (int s = 0; s < nactive; s++) m = fmaxf(m, __ldcg(base + (size_t)s * rec + G * hd + g));
                float num = 0.f, den = 0.f;
                for (int s = 0; s < nactive; s++) {
                    const float w = __expf(__ldcg(base + (size_t)s * rec + G * hd + g) - m);
                    num = fmaf(w, __ldcg(base + (size_t)s * rec + idx), num);
                    den = fmaf(w, __ldcg(base + (size_t)s * rec + G * hd + G + g), den);
                }
                op[idx] = __float2half_rn(den > 0.f ? num / den : 0.f);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Single-token step: rotary embedding, cache append and attention in one launch
// ---------------------------------------------------------------------------
// What the reference does with rope_forward, copy_to_kv_cache and attention_forward
// (src/transformer.cpp:225-245) for one new token.  Grid (splits, KV heads); a CTA owns
// 64 cache positions of one KV head and the query heads that share it.  After the
// dependency wait the CTA immediately requests its slice of K and V (bulk copies of the
// positions written by earlier steps), and while they fly it rotates the group's queries
// into shared memory; the CTA whose slice holds the new position also rotates the new key,
// puts key and value into its shared-memory slice and appends them to the cache.  Scores and
// softmax as in attention_kernel; P.V runs with one thread per (head, channel pair) and
// several position groups in parallel, reduced through shared memory.  Splits merge through
// the last-arriver scheme of attention_kernel.
constexpr int kDecChunk = 64;
constexpr int kDecMaxItems = 8;       // (head, channel pair) items per thread

struct DecodeArgs {
    half* q;                   // [n_heads, hd] of the new token, rotated in shared memory only
    const half* k;             // [n_kv_heads, hd] new key (unrotated)
    const half* v;             // [n_kv_heads, hd] new value
    half* k_cache;
    half* v_cache;
    half* out;                 // [n_heads, hd]
    int n_heads, n_kv_heads, head_dim, kv_len_max;
    int pos;                   // position of the new token (pos_dev overrides)
    const int* pos_dev;
    float theta;
    int nsplit;
    float* ws;
    unsigned* counters;
    int* err;
};

// kLong: built with the staged merge for more than 16 splits (a cache of more than 1024
// positions); the short instantiation is the kernel without it (fewer registers, and measured
// quicker on short caches).
template <bool kLong>
__global__ void __launch_bounds__(kAttnThreads)
attention_decode_kernel(const DecodeArgs a)
{
    extern __shared__ __align__(16) float smem[];
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hd = a.head_dim, hp = hd >> 1;
    const int G = a.n_heads / a.n_kv_heads;
    const int split = blockIdx.x, kvh = blockIdx.y;

    half* ks = reinterpret_cast<half*>(smem);                     // [kDecChunk][hd]
    half* vs = ks + kDecChunk * hd;                               // [kDecChunk][hd]
    float* qs = reinterpret_cast<float*>(vs + kDecChunk * hd);    // [G][hd]
    float* ps = qs + G * hd;                                      // [G][kDecChunk]
    float* m_run = ps + G * kDecChunk;
    float* l_run = m_run + kAttnMaxGroup;
    float* corr = l_run + kAttnMaxGroup;
    float* red = corr + kAttnMaxGroup;                            // P.V partials [groups][G*hd]
    __shared__ int s_last;
    __shared__ int s_ok;
    __shared__ __align__(8) unsigned long long s_bar;
    const uint32_t bar = smem_u32(&s_bar);
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // rotation frequency of this thread's channel pairs (independent of the position)
    const int npairs = G * hp;                                    // query pairs of the group
    float freq[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
        const int pr = (tid + u * kAttnThreads) % hp;
        freq[u] = 1.0f / powf(a.theta, (2.0f * (float)pr) / (float)hd);
    }
    __syncthreads();

    pdl_wait();
    const int pos = a.pos_dev ? *a.pos_dev : a.pos;
    const int limit = pos + 1;
    int nactive = (limit + kDecChunk - 1) / kDecChunk;
    if (nactive > a.nsplit) nactive = a.nsplit;
    if (split >= nactive) return;
    const int lo = split * kDecChunk;
    const int hi = (split == nactive - 1) ? limit : lo + kDecChunk;
    const bool owns_new = (split == nactive - 1);                 // this CTA's range ends with the new position

    const size_t cache_base = (size_t)kvh * (size_t)a.kv_len_max * hd;
    half* kb = a.k_cache + cache_base;
    half* vb = a.v_cache + cache_base;
    const float scale = rsqrtf((float)hd);

    const int items = G * hp;                                     // (head, channel pair) outputs
    const int pgroups = (items < kAttnThreads) ? kAttnThreads / items : 1;
    const int nitem = (items + kAttnThreads - 1) / kAttnThreads;  // items per thread when pgroups == 1
    float2 o[kDecMaxItems];
#pragma unroll
    for (int e = 0; e < kDecMaxItems; e++) o[e] = make_float2(0.f, 0.f);
    if (tid < G) {
        m_run[tid] = -FLT_MAX;
        l_run[tid] = 0.f;
    }

    uint32_t phase = 0;
    for (int c0 = lo; c0 < hi; c0 += kDecChunk) {
        const int nc = min(kDecChunk, hi - c0);
        const bool has_new = owns_new && (c0 + nc == limit);
        const int nold = has_new ? nc - 1 : nc;                   // positions that come from the cache
        if (tid == 0 && nold > 0) {
            const uint32_t bytes = (uint32_t)nold * hd * sizeof(half);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(2 * bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(ks)), "l"(kb + (size_t)c0 * hd), "r"(bytes), "r"(bar) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(vs)), "l"(vb + (size_t)c0 * hd), "r"(bytes), "r"(bar) : "memory");
        }
        if (c0 == lo) {
            // queries: rotate, scale, keep in shared memory (the global q is left as it was)
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = tid + u * kAttnThreads;
                if (i < npairs) {
                    const int g = i / hp, pr = i - g * hp;
                    const float2 x = __half22float2(*(reinterpret_cast<const half2*>(a.q + ((size_t)kvh * G + g) * hd) + pr));
                    float sn, cs;
                    sincosf((float)pos * freq[u], &sn, &cs);
                    // rounded to FP16 like the rotated q the reference stores, then scaled
                    qs[g * hd + 2 * pr] = __half2float(__float2half_rn(x.x * cs - x.y * sn)) * scale;
                    qs[g * hd + 2 * pr + 1] = __half2float(__float2half_rn(x.x * sn + x.y * cs)) * scale;
                }
            }
        }
        if (has_new && tid < hp) {
            // the new key (rotated) and value: into this slice and appended to the cache
            const float2 x = __half22float2(*(reinterpret_cast<const half2*>(a.k + (size_t)kvh * hd) + tid));
            float sn, cs;
            sincosf((float)pos * (1.0f / powf(a.theta, (2.0f * (float)tid) / (float)hd)), &sn, &cs);
            const half2 kr = __halves2half2(__float2half_rn(x.x * cs - x.y * sn), __float2half_rn(x.x * sn + x.y * cs));
            const half2 vr = *(reinterpret_cast<const half2*>(a.v + (size_t)kvh * hd) + tid);
            *(reinterpret_cast<half2*>(ks + (size_t)(nc - 1) * hd) + tid) = kr;
            *(reinterpret_cast<half2*>(vs + (size_t)(nc - 1) * hd) + tid) = vr;
            if (pos < a.kv_len_max) {
                *(reinterpret_cast<half2*>(kb + (size_t)pos * hd) + tid) = kr;
                *(reinterpret_cast<half2*>(vb + (size_t)pos * hd) + tid) = vr;
            }
        }
        if (tid == 0) s_ok = (nold > 0) ? (mbar_wait_bounded(bar, phase) ? 1 : 0) : 1;
        if (nold > 0) phase ^= 1u;
        __syncthreads();
        if (!s_ok) {
            if (tid == 0 && a.err) atomicExch(a.err, TLLM_ERR_TIMEOUT);
            return;
        }
        // ---- scores: thread <-> (position group, head g, 8-channel piece c) -------------
        // The thread keeps its piece of the (rotated, scaled) query in registers and walks the
        // positions of its group: one 16-byte K load and 8 FMAs per position, then the pieces of
        // a row are added with shuffles.  The lanes of a piece group read one full K row.
        {
            const int cpr = hd >> 3;                       // pieces per row (4, 8 or 16)
            const int tpg = G * cpr;                       // threads per position group
            const int c = tid % cpr, g = (tid / cpr) % G, pgp = tid / tpg, npg = kAttnThreads / tpg;
            const bool act = pgp < npg;               // threads beyond the last whole group only take part in the shuffles
            {
                const float4 q0 = *reinterpret_cast<const float4*>(qs + g * hd + c * 8);
                const float4 q1 = *reinterpret_cast<const float4*>(qs + g * hd + c * 8 + 4);
                auto piece = [&](int j) -> float {        // this thread's 8 channels of position j
                    if (!act || j >= nc) return 0.f;
                    const uint4 raw = *(reinterpret_cast<const uint4*>(ks + (size_t)j * hd) + c);
                    const half2* h = reinterpret_cast<const half2*>(&raw);
                    const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]);
                    const float2 f2 = __half22float2(h[2]), f3 = __half22float2(h[3]);
                    return (f0.x * q0.x + f0.y * q0.y) + (f1.x * q0.z + f1.y * q0.w) +
                           (f2.x * q1.x + f2.y * q1.y) + (f3.x * q1.z + f3.y * q1.w);
                };
                // four positions per trip: their loads and shuffle chains are independent
                // (the trip count must not depend on the position group: lanes of several groups can
                // share a warp and the shuffles below name all 32 lanes)
                for (int jb = 0; jb < nc; jb += 4 * npg) {
                    const int j0 = jb + pgp;
                    float d0 = piece(j0), d1 = piece(j0 + npg), d2 = piece(j0 + 2 * npg), d3 = piece(j0 + 3 * npg);
                    for (int o2 = cpr >> 1; o2 > 0; o2 >>= 1) {
                        d0 += __shfl_xor_sync(0xffffffffu, d0, o2);
                        d1 += __shfl_xor_sync(0xffffffffu, d1, o2);
                        d2 += __shfl_xor_sync(0xffffffffu, d2, o2);
                        d3 += __shfl_xor_sync(0xffffffffu, d3, o2);
                    }
                    if (c == 0 && act) {
                        float* pg_ = ps + g * kDecChunk;
                        if (j0 < nc) pg_[j0] = d0;
                        if (j0 + npg < nc) pg_[j0 + npg] = d1;
                        if (j0 + 2 * npg < nc) pg_[j0 + 2 * npg] = d2;
                        if (j0 + 3 * npg < nc) pg_[j0 + 3 * npg] = d3;
                    }
                }
            }
        }
        __syncthreads();
        for (int g = warp; g < G; g += kAttnThreads / 32) {
            float* p = ps + g * kDecChunk;
            float mx = -FLT_MAX;
            for (int j = lane; j < nc; j += 32) mx = fmaxf(mx, p[j]);
            mx = warp_max(mx);
            const float m_old = m_run[g];
            const float m_new = fmaxf(m_old, mx);
            float sum = 0.f;
            for (int j = lane; j < nc; j += 32) {
                const float e = __expf(p[j] - m_new);
                p[j] = e;
                sum += e;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float c = __expf(m_old - m_new);
                corr[g] = c;
                l_run[g] = l_run[g] * c + sum;
                m_run[g] = m_new;
            }
        }
        __syncthreads();
        // ---- P.V: thread <-> (head, channel pair) x position group ---------------------
        if (pgroups > 1) {
            const int item = tid % items, pg = tid / items;
            if (pg < pgroups) {
                const int g = item / hp, pr = item - g * hp;
                const float* p = ps + g * kDecChunk;
                const half2* vp = reinterpret_cast<const half2*>(vs) + pr;
                float2 acc = make_float2(o[0].x * corr[g], o[0].y * corr[g]);
                float2 acc1 = make_float2(0.f, 0.f), acc2 = acc1, acc3 = acc1;
                int j = pg;
                for (; j + 3 * pgroups < nc; j += 4 * pgroups) {
                    const half2 h0 = vp[(size_t)j * hp], h1 = vp[(size_t)(j + pgroups) * hp];
                    const half2 h2 = vp[(size_t)(j + 2 * pgroups) * hp], h3 = vp[(size_t)(j + 3 * pgroups) * hp];
                    const float p0 = p[j], p1 = p[j + pgroups], p2 = p[j + 2 * pgroups], p3 = p[j + 3 * pgroups];
                    const float2 v0 = __half22float2(h0), v1 = __half22float2(h1), v2 = __half22float2(h2), v3 = __half22float2(h3);
                    acc.x = fmaf(p0, v0.x, acc.x);
                    acc.y = fmaf(p0, v0.y, acc.y);
                    acc1.x = fmaf(p1, v1.x, acc1.x);
                    acc1.y = fmaf(p1, v1.y, acc1.y);
                    acc2.x = fmaf(p2, v2.x, acc2.x);
                    acc2.y = fmaf(p2, v2.y, acc2.y);
                    acc3.x = fmaf(p3, v3.x, acc3.x);
                    acc3.y = fmaf(p3, v3.y, acc3.y);
                }
                for (; j < nc; j += pgroups) {
                    const float2 vv = __half22float2(vp[(size_t)j * hp]);
                    acc.x = fmaf(p[j], vv.x, acc.x);
                    acc.y = fmaf(p[j], vv.y, acc.y);
                }
                o[0] = make_float2((acc.x + acc1.x) + (acc2.x + acc3.x), (acc.y + acc1.y) + (acc2.y + acc3.y));
            }
        } else {
#pragma unroll
            for (int e = 0; e < kDecMaxItems; e++) {
                const int item = e * kAttnThreads + tid;
                if (e < nitem && item < items) {
                    const int g = item / hp, pr = item - g * hp;
                    const float* p = ps + g * kDecChunk;
                    const half2* vp = reinterpret_cast<const half2*>(vs) + pr;
                    float2 acc = make_float2(o[e].x * corr[g], o[e].y * corr[g]);
                    float2 acc1 = make_float2(0.f, 0.f);
                    int j = 0;
                    for (; j + 1 < nc; j += 2) {
                        const float2 v0 = __half22float2(vp[(size_t)j * hp]), v1 = __half22float2(vp[(size_t)(j + 1) * hp]);
                        acc.x = fmaf(p[j], v0.x, acc.x);
                        acc.y = fmaf(p[j], v0.y, acc.y);
                        acc1.x = fmaf(p[j + 1], v1.x, acc1.x);
                        acc1.y = fmaf(p[j + 1], v1.y, acc1.y);
                    }
                    if (j < nc) {
                        const float2 vv = __half22float2(vp[(size_t)j * hp]);
                        acc.x = fmaf(p[j], vv.x, acc.x);
                        acc.y = fmaf(p[j], vv.y, acc.y);
                    }
                    o[e] = make_float2(acc.x + acc1.x, acc.y + acc1.y);
                }
            }
        }
        __syncthreads();
    }

    // ---- reduce the position groups, then write or publish ------------------------------
    if (pgroups > 1) {
        const int item = tid % items, pg = tid / items;
        if (pg < pgroups && pg > 0) *reinterpret_cast<float2*>(red + ((size_t)(pg - 1) * items + item) * 2) = o[0];
        __syncthreads();
        if (pg == 0)
            for (int r = 0; r < pgroups - 1; r++) {
                const float2 t = *reinterpret_cast<const float2*>(red + ((size_t)r * items + item) * 2);
                o[0].x += t.x;
                o[0].y += t.y;
            }
    }
    const bool writer_all = (pgroups == 1);
    half* op = a.out + (size_t)kvh * G * hd;
    const int rec = G * (hd + 2);
    float* my = a.ws + ((size_t)kvh * a.nsplit + split) * rec;
#pragma unroll
    for (int e = 0; e < kDecMaxItems; e++) {
        const int item = writer_all ? e * kAttnThreads + tid : tid;
        const bool mine = writer_all ? (e < nitem && item < items) : (e == 0 && tid < items);
        if (mine) {
            const int g = item / hp, pr = item - g * hp;
            if (nactive == 1) {
                const float l = l_run[g];
                const float inv = l > 0.f ? 1.0f / l : 0.f;
                *(reinterpret_cast<half2*>(op + (size_t)g * hd) + pr) =
                    __halves2half2(__float2half_rn(o[e].x * inv), __float2half_rn(o[e].y * inv));
            } else {
                *reinterpret_cast<float2*>(my + (size_t)g * hd + 2 * pr) = o[e];
            }
        }
    }
    if (nactive == 1) return;
    if (tid < G) {
        my[G * hd + tid] = m_run[tid];
        my[G * hd + G + tid] = l_run[tid];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned* cnt = a.counters + kvh;
        s_last = (atomicAdd(cnt, 1u) == (unsigned)(nactive - 1)) ? 1 : 0;
        if (s_last) *cnt = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float* base = a.ws + (size_t)kvh * a.nsplit * rec;
    if (kLong && nactive > 16 && (rec & 3) == 0 && (hd & 3) == 0 &&
        nactive * 2 * G * (int)sizeof(float) <= 2 * kDecChunk * hd * (int)sizeof(half)) {
        // Many splits (a long cache; with 16 or fewer the loop below is quicker, measured on the
        // 1B decode step: 0.632 against 0.651 ms per token).  A load from another SM's record
        // takes most of a microsecond, so the merge is built around loads in flight: the splits' (max, sum) pairs go to shared memory first (the
        // K/V slices there are no longer needed), then every thread owns four channels of one
        // head and requests their partial outputs of sixteen splits at a time.
        float* s_ml = smem;                                    // [nactive][2 * G]
        for (int i = tid; i < nactive * 2 * G; i += kAttnThreads) {
            const int sp = i / (2 * G), j = i - sp * 2 * G;
            s_ml[i] = __ldcg(base + (size_t)sp * rec + G * hd + j);
        }
        __syncthreads();
        for (int i4 = tid; i4 < (G * hd) >> 2; i4 += kAttnThreads) {
            const int g = (i4 << 2) / hd;
            float mx = -FLT_MAX;
            for (int sp = 0; sp < nactive; sp++) mx = fmaxf(mx, s_ml[sp * 2 * G + g]);
            float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
            float den = 0.f;
            for (int s0 = 0; s0 < nactive; s0 += 16) {
                float4 os[16];
#pragma unroll
                for (int u = 0; u < 16; u++)
                    os[u] = __ldcg(reinterpret_cast<const float4*>(base + (size_t)min(s0 + u, nactive - 1) * rec) + i4);
#pragma unroll
                for (int u = 0; u < 16; u++) {
                    if (s0 + u < nactive) {
                        const float w = __expf(s_ml[(s0 + u) * 2 * G + g] - mx);
                        num.x = fmaf(w, os[u].x, num.x);
                        num.y = fmaf(w, os[u].y, num.y);
                        num.z = fmaf(w, os[u].z, num.z);
                        num.w = fmaf(w, os[u].w, num.w);
                        den = fmaf(w, s_ml[(s0 + u) * 2 * G + G + g], den);
                    }
                }
            }
            const float inv = den > 0.f ? 1.0f / den : 0.f;
            half2* o2 = reinterpret_cast<half2*>(op + (size_t)(i4 << 2));
            o2[0] = __halves2half2(__float2half_rn(num.x * inv), __float2half_rn(num.y * inv));
            o2[1] = __halves2half2(__float2half_rn(num.z * inv), __float2half_rn(num.w * inv));
        }
        return;
    }
    for (int idx = tid; idx < G * hd; idx += kAttnThreads) {
        const int g = idx / hd;
        float m = -FLT_MAX, num = 0.f, den = 0.f;
        for (int s0 = 0; s0 < nactive; s0 += 8) {
            // issue every load of up to eight splits before any of them is used
            float ms[8], ls[8], os[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const bool live = s0 + u < nactive;
                const float* r = base + (size_t)(live ? s0 + u : s0) * rec;
                ms[u] = live ? __ldcg(r + G * hd + g) : -FLT_MAX;
                ls[u] = live ? __ldcg(r + G * hd + G + g) : 0.f;
                os[u] = live ? __ldcg(r + idx) : 0.f;
            }
            float mx = m;
#pragma unroll
            for (int u = 0; u < 8; u++) mx = fmaxf(mx, ms[u]);
            const float c0 = __expf(m - mx);              // rescale what earlier trips accumulated
            num *= c0;
            den *= c0;
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const float w = __expf(ms[u] - mx);      // 0 for the padding entries
                num = fmaf(w, os[u], num);
                den = fmaf(w, ls[u], den);
            }
            m = mx;
        }
        op[idx] = __float2half_rn(den > 0.f ? num / den : 0.f);
    }
}

size_t attention_decode_workspace_bytes(int n_heads, int n_kv_heads, int head_dim, int kv_len_max)
{
    const int G = n_heads / n_kv_heads;
    const int nsplit = (kv_len_max + kDecChunk - 1) / kDecChunk;
    return (size_t)n_kv_heads * nsplit * G * (head_dim + 2) * sizeof(float);
}

// One new token at position pos (or *pos_dev): q [n_heads, hd], k and v [n_kv_heads, hd] as
// the projections wrote them; the rotated key and the value are appended to the caches.
// ws: attention_decode_workspace_bytes; counters: n_kv_heads zero-initialised unsigned.
int launch_attention_decode(half* q, const half* k, const half* v, half* k_cache, half* v_cache, half* out, int n_heads,
                            int n_kv_heads, int head_dim, int kv_len_max, int pos, const int* pos_dev, float theta,
                            float* ws, unsigned* counters, cudaStream_t stream)
{
    if (n_kv_heads <= 0 || n_heads % n_kv_heads) return fail(TLLM_ERR_SHAPE, "attention: n_heads=%d n_kv_heads=%d", n_heads, n_kv_heads);
    const int G = n_heads / n_kv_heads;
    const int items = G * head_dim / 2;
    const int cpr = head_dim / 8;
    if (G > kAttnMaxGroup || head_dim % 8 || head_dim > 128 || (cpr & (cpr - 1)) || cpr < 2 || G * cpr > kAttnThreads ||
        items > kDecMaxItems * kAttnThreads || G * head_dim / 2 > 4 * kAttnThreads)
        return fail(TLLM_ERR_SHAPE, "attention: head_dim=%d with %d heads per group is not supported", head_dim, G);
    if (!pos_dev && (pos < 0 || pos >= kv_len_max)) return fail(TLLM_ERR_SHAPE, "attention: pos=%d kv_len_max=%d", pos, kv_len_max);
    DecodeArgs a = {};
    a.q = q;
    a.k = k;
    a.v = v;
    a.k_cache = k_cache;
    a.v_cache = v_cache;
    a.out = out;
    a.n_heads = n_heads;
    a.n_kv_heads = n_kv_heads;
    a.head_dim = head_dim;
    a.kv_len_max = kv_len_max;
    a.pos = pos;
    a.pos_dev = pos_dev;
    a.theta = theta;
    a.nsplit = (kv_len_max + kDecChunk - 1) / kDecChunk;
    a.ws = ws;
    a.counters = counters;
    a.err = device_error_flag();
    const int pgroups = (items < kAttnThreads) ? kAttnThreads / items : 1;
    const size_t smem = (size_t)2 * kDecChunk * head_dim * sizeof(half) +
                        ((size_t)G * head_dim + (size_t)G * kDecChunk + 3 * kAttnMaxGroup +
                         (size_t)(pgroups > 1 ? (pgroups - 1) * items * 2 : 0)) * sizeof(float);
    static bool attr[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr[dev]) {
        cudaFuncSetAttribute(attention_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(attention_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr[dev] = true;
    }
    if (a.nsplit > 16)
        return launch_pdl("attention_decode", attention_decode_kernel<true>, dim3(a.nsplit, n_kv_heads), dim3(kAttnThreads),
                          smem, stream, a);
    return launch_pdl("attention_decode", attention_decode_kernel<false>, dim3(a.nsplit, n_kv_heads), dim3(kAttnThreads), smem,
                      stream, a);
}

size_t attention_workspace_bytes(int batch, int n_heads, int n_kv_heads, int head_dim, int kv_len_max)
{
    const int G = n_heads / n_kv_heads;
    const int nsplit = (kv_len_max + kAttnChunk - 1) / kAttnChunk;
    return (size_t)batch * n_kv_heads * nsplit * G * (head_dim + 2) * sizeof(float);
}

// ws / counters: decode scratch (attention_workspace_bytes; counters zero-initialised,
// batch * n_kv_heads unsigned).  With ws == nullptr decode runs as one CTA per KV head.
int launch_attention(const half* q, const half* k_cache, const half* v_cache, half* out, int batch, int n_heads,
                     int n_kv_heads, int head_dim, int seq_len, int kv_len, int kv_len_max, const int* kv_len_dev,
                     float* ws, unsigned* counters, cudaStream_t stream)
{
    if (batch == 0 || seq_len == 0) return TLLM_OK;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads) return fail(TLLM_ERR_SHAPE, "attention: n_heads=%d n_kv_heads=%d", n_heads, n_kv_heads);
    const int G = n_heads / n_kv_heads;
    if (G > kAttnMaxGroup) return fail(TLLM_ERR_SHAPE, "attention: %d query heads per KV head (limit %d)", G, kAttnMaxGroup);
    if (head_dim % 8 || head_dim > 128 || G * head_dim > kAttnMaxElems * kAttnThreads)
        return fail(TLLM_ERR_SHAPE, "attention: head_dim=%d (a multiple of 8 up to 128) with %d heads per group is not supported",
                    head_dim, G);
    if (!kv_len_dev && (kv_len < seq_len || kv_len > kv_len_max))
        return fail(TLLM_ERR_SHAPE, "attention: kv_len=%d seq_len=%d kv_len_max=%d", kv_len, seq_len, kv_len_max);
    AttnArgs a = {};
    a.q = q;
    a.k_cache = k_cache;
    a.v_cache = v_cache;
    a.out = out;
    a.n_heads = n_heads;
    a.n_kv_heads = n_kv_heads;
    a.head_dim = head_dim;
    a.seq_len = seq_len;
    a.kv_len = kv_len;
    a.kv_len_max = kv_len_max;
    a.kv_len_dev = kv_len_dev;
    a.ws = ws;
    a.counters = counters;
    const bool decode = (seq_len == 1);
    a.nsplit = (decode && ws) ? (kv_len_max + kAttnChunk - 1) / kAttnChunk : 1;
    a.err = device_error_flag();
    const size_t smem = (size_t)2 * kAttnChunk * head_dim * sizeof(half) +
                        ((size_t)G * head_dim + (size_t)G * kAttnChunk + 3 * kAttnMaxGroup) * sizeof(float);
    static bool attr[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr[dev]) {
        cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr[dev] = true;
    }
    const dim3 grid(decode ? a.nsplit : seq_len, n_kv_heads, batch);
    return launch_pdl("attention", attention_kernel, grid, dim3(kAttnThreads), smem, stream, a);
}

}  // namespace tllm

