// extern "C" entry points of the layer operators (include/tllm_b200_layer.h):
// argument checks and dispatch to layer_ops.cu / attention.cu.
#include <mutex>

#include "layer.cuh"
#include "tllm_b200_layer.h"

using namespace tllm;

namespace {
inline bool misaligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; }
inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }

// Scratch of the single-token attention called through the C ABI: the partial results of the
// splits over cache positions and the per-(sequence, KV head) arrival counters.  One buffer per
// device, grown on demand; it cannot grow while the stream is being captured into a graph.
struct AttnScratch {
    float* ws = nullptr;
    size_t ws_bytes = 0;
    unsigned* counters = nullptr;
    size_t n_counters = 0;
};
AttnScratch g_attn[64];
std::mutex g_attn_mu;

int attention_scratch(size_t ws_bytes, size_t n_counters, cudaStream_t stream, float** ws, unsigned** counters)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(TLLM_ERR_LAUNCH, "attention: no current device");
    std::lock_guard<std::mutex> lk(g_attn_mu);
    AttnScratch& s = g_attn[dev];
    if (s.ws_bytes < ws_bytes || s.n_counters < n_counters) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(stream, &cap);
        if (cap != cudaStreamCaptureStatusNone)
            return fail(TLLM_ERR_LAUNCH, "attention: the split workspace must grow (%zu bytes); call once with these sizes "
                        "outside stream capture first", ws_bytes);
        if (cudaDeviceSynchronize() != cudaSuccess) return fail(TLLM_ERR_LAUNCH, "attention: device synchronize failed");
        if (s.ws) cudaFree(s.ws);
        if (s.counters) cudaFree(s.counters);
        s = AttnScratch();
        const size_t nb = ws_bytes > s.ws_bytes ? ws_bytes : s.ws_bytes, nc = n_counters > 64 ? n_counters : 64;
        if (cudaMalloc(&s.ws, nb) != cudaSuccess || cudaMalloc(&s.counters, nc * sizeof(unsigned)) != cudaSuccess ||
            cudaMemset(s.counters, 0, nc * sizeof(unsigned)) != cudaSuccess) {
            cudaGetLastError();
            if (s.ws) cudaFree(s.ws);
            if (s.counters) cudaFree(s.counters);
            s = AttnScratch();
            return fail(TLLM_ERR_LAUNCH, "attention: cannot allocate %zu bytes of split workspace", nb);
        }
        s.ws_bytes = nb;
        s.n_counters = nc;
    }
    *ws = s.ws;
    *counters = s.counters;
    return TLLM_OK;
}
}  // namespace

extern "C" {

int tllm_b200_rmsnorm(const void* input, const void* weight, void* output, const void* residual, void* residual_out,
                      int batch, int dim, float eps, void* stream)
{
    if (!input || !weight || !output) return fail(TLLM_ERR_NULL, "rmsnorm: null pointer");
    if (batch < 0 || dim < 1) return fail(TLLM_ERR_SHAPE, "rmsnorm: batch=%d dim=%d", batch, dim);
    int st = check_device();
    if (st) return st;
    return launch_rmsnorm((const half*)input, (const half*)weight, (half*)output, (const half*)residual,
                          (half*)residual_out, nullptr, nullptr, batch, dim, eps, 0, S(stream));
}

static int check_heads(const char* fn, int batch, int seq_len, int n_heads, int n_kv_heads, int head_dim)
{
    if (batch < 0 || seq_len < 0 || n_heads < 0 || n_kv_heads < 0 || head_dim < 2 || (head_dim & 1))
        return fail(TLLM_ERR_SHAPE, "%s: batch=%d seq_len=%d heads=%d/%d head_dim=%d", fn, batch, seq_len, n_heads,
                    n_kv_heads, head_dim);
    return TLLM_OK;
}

int tllm_b200_rope(void* q, void* k, int batch, int seq_len, int n_heads, int n_kv_heads, int head_dim, int start_pos,
                   float theta, void* stream)
{
    if (!q || !k) return fail(TLLM_ERR_NULL, "rope: null pointer");
    int st = check_heads("rope", batch, seq_len, n_heads, n_kv_heads, head_dim);
    if (st || (st = check_device())) return st;
    if (misaligned(q, 4) || misaligned(k, 4)) return fail(TLLM_ERR_ALIGN, "rope: q and k must be 4-byte aligned");
    return launch_rope((half*)q, (half*)k, nullptr, nullptr, nullptr, batch, seq_len, n_heads, n_kv_heads, head_dim,
                       start_pos, nullptr, theta, 0, 1, S(stream));
}

int tllm_b200_copy_to_kv_cache(const void* k, const void* v, void* k_cache, void* v_cache, int batch, int n_kv_heads,
                               int head_dim, int seq_len, int start_pos, int max_seq_len, void* stream)
{
    if (!k || !v || !k_cache || !v_cache) return fail(TLLM_ERR_NULL, "copy_to_kv_cache: null pointer");
    int st = check_heads("copy_to_kv_cache", batch, seq_len, 0, n_kv_heads, head_dim);
    if (st || (st = check_device())) return st;
    if (misaligned(k, 4) || misaligned(v, 4) || misaligned(k_cache, 4) || misaligned(v_cache, 4))
        return fail(TLLM_ERR_ALIGN, "copy_to_kv_cache: pointers must be 4-byte aligned");
    return launch_rope(nullptr, (half*)k, (const half*)v, (half*)k_cache, (half*)v_cache, batch, seq_len, 0, n_kv_heads,
                       head_dim, start_pos, nullptr, 1.0f, max_seq_len, 0, S(stream));
}

int tllm_b200_rope_append(void* q, void* k, const void* v, void* k_cache, void* v_cache, int batch, int seq_len,
                          int n_heads, int n_kv_heads, int head_dim, int start_pos, float theta, int max_seq_len,
                          void* stream)
{
    if (!q || !k || !v || !k_cache || !v_cache) return fail(TLLM_ERR_NULL, "rope_append: null pointer");
    int st = check_heads("rope_append", batch, seq_len, n_heads, n_kv_heads, head_dim);
    if (st || (st = check_device())) return st;
    if (misaligned(q, 4) || misaligned(k, 4) || misaligned(v, 4) || misaligned(k_cache, 4) || misaligned(v_cache, 4))
        return fail(TLLM_ERR_ALIGN, "rope_append: pointers must be 4-byte aligned");
    return launch_rope((half*)q, (half*)k, (const half*)v, (half*)k_cache, (half*)v_cache, batch, seq_len, n_heads,
                       n_kv_heads, head_dim, start_pos, nullptr, theta, max_seq_len, 1, S(stream));
}

int tllm_b200_attention(const void* q, const void* k_cache, const void* v_cache, void* output, int batch, int n_heads,
                        int n_kv_heads, int head_dim, int seq_len, int kv_len, int kv_len_max, void* stream)
{
    if (!q || !k_cache || !v_cache || !output) return fail(TLLM_ERR_NULL, "attention: null pointer");
    if (batch < 0 || seq_len < 0 || n_heads < 1 || n_kv_heads < 1)
        return fail(TLLM_ERR_SHAPE, "attention: batch=%d seq_len=%d heads=%d/%d", batch, seq_len, n_heads, n_kv_heads);
    if (misaligned(k_cache, 16) || misaligned(v_cache, 2) || misaligned(q, 2))
        return fail(TLLM_ERR_ALIGN, "attention: k_cache must be 16-byte aligned");
    int st = check_device();
    if (st) return st;
    // one token per sequence over a long cache: split the cache positions over CTAs (a single
    // CTA per KV head walks 2048 positions in about 0.2 ms, far longer than the projections)
    float* ws = nullptr;
    unsigned* counters = nullptr;
    if (seq_len == 1 && batch > 0 && kv_len_max > 256 && n_heads % n_kv_heads == 0) {
        st = attention_scratch(attention_workspace_bytes(batch, n_heads, n_kv_heads, head_dim, kv_len_max),
                               (size_t)batch * n_kv_heads, S(stream), &ws, &counters);
        if (st) return st;
    }
    return launch_attention((const half*)q, (const half*)k_cache, (const half*)v_cache, (half*)output, batch, n_heads,
                            n_kv_heads, head_dim, seq_len, kv_len, kv_len_max, nullptr, ws, counters, S(stream));
}

int tllm_b200_attention_decode(void* q, const void* k, const void* v, void* k_cache, void* v_cache, void* output,
                               int n_heads, int n_kv_heads, int head_dim, int pos, float theta, int max_seq_len,
                               void* stream)
{
    if (!q || !k || !v || !k_cache || !v_cache || !output) return fail(TLLM_ERR_NULL, "attention_decode: null pointer");
    if (n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads || max_seq_len < 1)
        return fail(TLLM_ERR_SHAPE, "attention_decode: heads=%d/%d max_seq_len=%d", n_heads, n_kv_heads, max_seq_len);
    if (misaligned(k_cache, 16) || misaligned(v_cache, 16) || misaligned(q, 4) || misaligned(k, 4) || misaligned(v, 4))
        return fail(TLLM_ERR_ALIGN, "attention_decode: caches must be 16-byte aligned, q/k/v 4-byte aligned");
    int st = check_device();
    if (st) return st;
    float* ws = nullptr;
    unsigned* counters = nullptr;
    st = attention_scratch(attention_decode_workspace_bytes(n_heads, n_kv_heads, head_dim, max_seq_len), (size_t)n_kv_heads,
                           S(stream), &ws, &counters);
    if (st) return st;
    return launch_attention_decode((half*)q, (const half*)k, (const half*)v, (half*)k_cache, (half*)v_cache, (half*)output,
                                   n_heads, n_kv_heads, head_dim, max_seq_len, pos, nullptr, theta, ws, counters, S(stream));
}

int tllm_b200_silu_mul(const void* gate, const void* up, void* output, int size, void* stream)
{
    if (!gate || !up || !output) return fail(TLLM_ERR_NULL, "silu_mul: null pointer");
    if (size < 0) return fail(TLLM_ERR_SHAPE, "silu_mul: size=%d", size);
    if (misaligned(gate, 4) || misaligned(up, 4) || misaligned(output, 4))
        return fail(TLLM_ERR_ALIGN, "silu_mul: pointers must be 4-byte aligned");
    int st = check_device();
    if (st) return st;
    return launch_silu_mul((const half*)gate, (const half*)up, (half*)output, size, nullptr, nullptr, S(stream));
}

int tllm_b200_add(const void* a, const void* b, void* output, int size, void* stream)
{
    if (!a || !b || !output) return fail(TLLM_ERR_NULL, "add: null pointer");
    if (size < 0) return fail(TLLM_ERR_SHAPE, "add: size=%d", size);
    if (misaligned(a, 4) || misaligned(b, 4) || misaligned(output, 4))
        return fail(TLLM_ERR_ALIGN, "add: pointers must be 4-byte aligned");
    int st = check_device();
    if (st) return st;
    return launch_add((const half*)a, (const half*)b, (half*)output, size, S(stream));
}

int tllm_b200_embedding_lookup(const void* table, const int* indices, void* output, int n_tokens, int dim, void* stream)
{
    if (!table || !indices || !output) return fail(TLLM_ERR_NULL, "embedding_lookup: null pointer");
    if (n_tokens < 0 || dim < 1) return fail(TLLM_ERR_SHAPE, "embedding_lookup: n_tokens=%d dim=%d", n_tokens, dim);
    int st = check_device();
    if (st) return st;
    return launch_embedding((const half*)table, indices, (half*)output, n_tokens, dim, S(stream));
}

int tllm_b200_fp16_gemv(const void* weight, const void* input, void* output, int rows, int cols, void* stream)
{
    if (!weight || !input || !output) return fail(TLLM_ERR_NULL, "fp16_gemv: null pointer");
    if (rows < 0 || cols < 1) return fail(TLLM_ERR_SHAPE, "fp16_gemv: rows=%d cols=%d", rows, cols);
    int st = check_device();
    if (st) return st;
    return launch_fp16_gemv((const half*)weight, (const half*)input, (half*)output, rows, cols, S(stream));
}

int tllm_b200_fp16_gemm(const void* A, const void* B, void* C, int M, int N, int K, void* stream)
{
    if (!A || !B || !C) return fail(TLLM_ERR_NULL, "fp16_gemm: null pointer");
    if (M < 0 || N < 0 || K < 1) return fail(TLLM_ERR_SHAPE, "fp16_gemm: M=%d N=%d K=%d", M, N, K);
    int st = check_device();
    if (st) return st;
    return launch_fp16_gemm((const half*)A, (const half*)B, (half*)C, M, N, K, S(stream));
}

int tllm_b200_gemv_int8_packed_multi(int count, const void* const* packed, void* const* y, const int* rows, int cols,
                                     const void* x_int8, const float* input_scale_dev, void* stream)
{
    if (!packed || !y || !rows || !x_int8 || !input_scale_dev) return fail(TLLM_ERR_NULL, "gemv_int8_packed_multi: null pointer");
    if (count < 1 || count > TLLM_MAX_FUSED) return fail(TLLM_ERR_BATCH, "count %d outside 1..%d", count, TLLM_MAX_FUSED);
    if (cols < kGroup || cols % kGroup) return fail(TLLM_ERR_SHAPE, "cols=%d: need a positive multiple of 128", cols);
    if (misaligned(x_int8, 16)) return fail(TLLM_ERR_ALIGN, "x_int8 must be 16-byte aligned");
    for (int i = 0; i < count; i++) {
        if (!packed[i] || !y[i]) return fail(TLLM_ERR_NULL, "gemv_int8_packed_multi: null pointer in table");
        if (rows[i] < 1) return fail(TLLM_ERR_SHAPE, "rows[%d]=%d", i, rows[i]);
        if (misaligned(packed[i], 16)) return fail(TLLM_ERR_ALIGN, "packed weights must be 16-byte aligned");
    }
    int st = check_device();
    if (st) return st;
    return launch_gemv_int8_packed_multi(count, (const uint8_t* const*)packed, (half* const*)y, rows, cols,
                                         (const int8_t*)x_int8, input_scale_dev, S(stream));
}

}  // extern "C"
