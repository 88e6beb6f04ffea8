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
// positions in chunks of 256 with an online softmax:
//   scores  - one thread per position, dot products against the group's query heads
//             (queries pre-scaled in shared memory), 128-bit K loads;
//   softmax - one warp per query head over the chunk's 256 scores;
//   P.V     - one thread per (query head, channel), V rows read coalesced.
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

    float* qs = smem;                         // [G][hd] queries times 1/sqrt(hd)
    float* ps = qs + G * hd;                  // [G][kAttnChunk] scores, then probabilities
    float* m_run = ps + G * kAttnChunk;       // [G] running maximum
    float* l_run = m_run + kAttnMaxGroup;     // [G] running sum
    float* corr = l_run + kAttnMaxGroup;      // [G] rescale factor of this chunk
    __shared__ int s_last;

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

    for (int c0 = lo; c0 < hi; c0 += kAttnChunk) {
        const int nc = min(kAttnChunk, hi - c0);
        // ---- scores: thread j <-> position c0 + j --------------------------------
        if (tid < nc) {
            float dot[kAttnMaxGroup];
#pragma unroll
            for (int g = 0; g < kAttnMaxGroup; g++) dot[g] = 0.f;
            const uint4* k4 = reinterpret_cast<const uint4*>(kb + (size_t)(c0 + tid) * hd);
            for (int d8 = 0; d8 < hd / 8; d8++) {
                const uint4 raw = __ldg(k4 + d8);
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
                    const half* vp = vb + (size_t)c0 * hd + d;
                    float acc = o[e] * corr[g];
                    int j = 0;
                    for (; j + 4 <= nc; j += 4) {
                        const float v0 = __half2float(vp[(size_t)(j + 0) * hd]);
                        const float v1 = __half2float(vp[(size_t)(j + 1) * hd]);
                        const float v2 = __half2float(vp[(size_t)(j + 2) * hd]);
                        const float v3 = __half2float(vp[(size_t)(j + 3) * hd]);
                        acc = fmaf(p[j], v0, acc);
                        acc = fmaf(p[j + 1], v1, acc);
                        acc = fmaf(p[j + 2], v2, acc);
                        acc = fmaf(p[j + 3], v3, acc);
                    }
                    for (; j < nc; j++) acc = fmaf(p[j], __half2float(vp[(size_t)j * hd]), acc);
                    o[e] = acc;
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
    if (head_dim % 8 || G * head_dim > kAttnMaxElems * kAttnThreads)
        return fail(TLLM_ERR_SHAPE, "attention: head_dim=%d with %d heads per group is not supported", head_dim, G);
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
    const size_t smem = ((size_t)G * head_dim + (size_t)G * kAttnChunk + 3 * kAttnMaxGroup) * sizeof(float);
    static bool attr[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr[dev]) {
        cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
        attr[dev] = true;
    }
    const dim3 grid(decode ? a.nsplit : seq_len, n_kv_heads, batch);
    return launch_pdl("attention", attention_kernel, grid, dim3(kAttnThreads), smem, stream, a);
}

}  // namespace tllm
