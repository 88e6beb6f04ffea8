// The reference engine's Transformer (src/transformer.cpp) on this library's kernels.
//
// forward() keeps the reference's order of operations and its choice of arithmetic --
// FP16 activations through the tensor-core GEMM for several tokens, INT8-quantised
// activations through the streaming GEMV for one token -- but a single-token step makes
// 5 launches per layer instead of 20 and never touches the host:
//   [q|k|v] GEMV whose staging phase does residual add + RMSNorm + quantise |
//   RoPE + cache append + attention (all query heads of a KV head per CTA, split over the
//   cache) | o GEMV with the quantiser in its staging |
//   [gate|up] GEMV with add + RMSNorm + quantise in its staging |
//   down GEMV with SwiGLU + quantise in its staging
// The activation scale stays in device memory (the reference copies it to the host before
// every GEMV, src/transformer.cpp:132-136), the position and the token live in device
// memory too, and greedy sampling runs on the device, so that one decode step can be
// captured as a CUDA graph and replayed.
#include <utility>
#include <vector>

#include "layer.cuh"
#include "tllm_b200_layer.h"

namespace tllm {

namespace {

struct PackedW {
    uint8_t* p = nullptr;
    int rows = 0, cols = 0;
};

struct LayerW {
    PackedW q, k, v, o, gate, up, down;
    // q,k,v and gate,up are packed back to back (their row counts are multiples of 16), so
    // that a single-token step streams each group as ONE matrix: [q|k|v] and [gate|up].
    PackedW qkv, gate_up;
    const half* attn_norm = nullptr;
    const half* ffn_norm = nullptr;
};

struct Decoder {
    tllm_b200_model_desc d = {};
    int flags = 0;
    std::vector<LayerW> layers;
    PackedW lm_head;
    // activations (max_seq_len rows where a prefill needs them)
    half *residual = nullptr, *hidden = nullptr, *hidden2 = nullptr, *q = nullptr, *k = nullptr, *v = nullptr;
    half *attn_out = nullptr, *gate = nullptr, *up = nullptr, *ffn_out = nullptr, *logits = nullptr;
    half *k_cache = nullptr, *v_cache = nullptr;
    half *qkv1 = nullptr, *gu1 = nullptr;      // single-token outputs of the concatenated matrices
    half* residual2 = nullptr;                 // second residual vector of the fused single-token step
    bool fused_ok = false;                     // every layer has concatenated q|k|v and gate|up
    int max_batch = 1;                         // sequences with their own KV cache
    int8_t* xq = nullptr;
    float* xscale = nullptr;
    float* attn_ws = nullptr;
    float* attn_ws2 = nullptr;     // split records of the fused single-token attention
    unsigned* attn_counters = nullptr;
    // device-side state of the graph-replayed decode loop
    int* state = nullptr;          // [0] token, [1] position, [2] step
    int* history = nullptr;        // generated tokens
    int history_cap = 0;
    float* am_val = nullptr;
    int* am_idx = nullptr;
    unsigned* am_counter = nullptr;
    cudaStream_t stream = nullptr; // owned, for generate()
    cudaGraphExec_t step_graph = nullptr;
    std::vector<void*> owned;
};

template <typename T>
int dev_alloc(Decoder* D, T** out, size_t n, bool zero)
{
    void* p = nullptr;
    const cudaError_t e = cudaMalloc(&p, n * sizeof(T));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(TLLM_ERR_LAUNCH, "decoder: cudaMalloc(%zu bytes): %s", n * sizeof(T), cudaGetErrorString(e));
    }
    if (zero) cudaMemset(p, 0, n * sizeof(T));
    D->owned.push_back(p);
    *out = static_cast<T*>(p);
    return TLLM_OK;
}

int check_weight(const tllm_b200_ternary_weight& w)
{
    if (!w.nonzero_masks || !w.sign_masks || !w.scales) return fail(TLLM_ERR_NULL, "decoder: null ternary weight");
    if (w.out_features < 1 || w.in_features < kGroup || w.in_features % kGroup)
        return fail(TLLM_ERR_SHAPE, "decoder: weight %d x %d: in_features must be a positive multiple of 128", w.out_features,
                    w.in_features);
    return TLLM_OK;
}

// dst == nullptr: allocate; else repack into dst (part of a concatenated buffer)
int pack(Decoder* D, const tllm_b200_ternary_weight& w, PackedW* out, cudaStream_t stream, uint8_t* dst = nullptr)
{
    int st = check_weight(w);
    if (st) return st;
    out->rows = w.out_features;
    out->cols = w.in_features;
    if (dst) out->p = dst;
    else if ((st = dev_alloc(D, &out->p, packed_bytes(w.out_features, w.in_features), false))) return st;
    return weight_prepare(static_cast<const uint32_t*>(w.nonzero_masks), static_cast<const uint32_t*>(w.sign_masks),
                          static_cast<const half*>(w.scales), w.out_features, w.in_features, out->p, stream);
}

// Packs `count` matrices with the same input width back to back; `all` views them as one.
int pack_group(Decoder* D, int count, const tllm_b200_ternary_weight* const* w, PackedW* const* out, PackedW* all,
               cudaStream_t stream)
{
    int st;
    size_t total = 0;
    int rows = 0;
    bool concat = true;
    for (int i = 0; i < count; i++) {
        if ((st = check_weight(*w[i]))) return st;
        concat = concat && (w[i]->out_features % packed_row_align() == 0) && (w[i]->in_features == w[0]->in_features);
        total += packed_bytes(w[i]->out_features, w[i]->in_features);
        rows += w[i]->out_features;
    }
    if (!concat) {
        *all = PackedW();
        for (int i = 0; i < count; i++)
            if ((st = pack(D, *w[i], out[i], stream))) return st;
        return TLLM_OK;
    }
    uint8_t* base = nullptr;
    if ((st = dev_alloc(D, &base, total, false))) return st;
    size_t off = 0;
    for (int i = 0; i < count; i++) {
        if ((st = pack(D, *w[i], out[i], stream, base + off))) return st;
        off += packed_bytes(w[i]->out_features, w[i]->in_features);
    }
    all->p = base;
    all->rows = rows;
    all->cols = w[0]->in_features;
    return TLLM_OK;
}

// y[n_tokens, rows] = x[n_tokens, cols] . W^T with FP16 activations: the tcgen05 GEMM for
// token batches, passes of the streaming GEMV for a few tokens.
int linear_f16(const PackedW& w, const half* x, half* y, int n_tokens, cudaStream_t stream)
{
    if (n_tokens > 8 && gemm_tcgen05_supported(n_tokens, w.rows, w.cols))
        return launch_gemm_tcgen05(x, w.p, y, n_tokens, w.rows, w.cols, stream);
    return launch_gemv_packed(w.p, x, y, n_tokens, w.rows, w.cols, stream);
}

int linear_multi(Decoder* D, int count, const PackedW* const* w, half* const* y, const half* x, bool int8,
                 int n_tokens, cudaStream_t stream)
{
    const uint8_t* p[TLLM_MAX_FUSED];
    int rows[TLLM_MAX_FUSED];
    for (int i = 0; i < count; i++) {
        p[i] = w[i]->p;
        rows[i] = w[i]->rows;
    }
    if (n_tokens == 1) {
        if (int8) return launch_gemv_int8_packed_multi(count, p, y, rows, w[0]->cols, D->xq, D->xscale, stream);
        return launch_gemv_packed_multi(count, p, y, rows, w[0]->cols, x, stream);
    }
    for (int i = 0; i < count; i++) {
        const int st = linear_f16(*w[i], x, y[i], n_tokens, stream);
        if (st) return st;
    }
    return TLLM_OK;
}

// One pass of the layer stack.
//   batch == 0: n tokens of sequence `seq` at positions start_pos.. (pos_dev != nullptr: one
//               token whose position is read from device memory, start_pos ignored);
//   batch  > 0: one token of each of the sequences 0..batch-1 (n == batch), all at position
//               start_pos, each against its own KV cache; logits for every sequence.
int forward(Decoder* D, const int* tokens, int n, int start_pos, const int* pos_dev, int seq, int batch, cudaStream_t s)
{
    const tllm_b200_model_desc& c = D->d;
    const int hidden = c.hidden_dim, inter = c.intermediate_dim, qdim = c.n_heads * c.head_dim;
    const bool i8 = (n == 1) && (D->flags & TLLM_DECODER_INT8_DECODE);
    const int bsz = batch > 0 ? batch : 1, seq_n = batch > 0 ? 1 : n;       // attention geometry
    const size_t kv_seq = (size_t)c.max_seq_len * c.n_kv_heads * c.head_dim;  // one sequence's cache of a layer
    const size_t kv_layer = kv_seq * D->max_batch;
    const size_t kv_first = batch > 0 ? 0 : (size_t)seq * kv_seq;
    int8_t* xq = i8 ? D->xq : nullptr;
    float* xs = i8 ? D->xscale : nullptr;
    int st;
#define TRY(x) do { if ((st = (x)) != TLLM_OK) return st; } while (0)
    TRY(launch_embedding(static_cast<const half*>(c.embedding_table), tokens, D->residual, n, hidden, s));
    half* res_cur = D->residual;
    if (i8 && D->fused_ok) {
        // Single token, INT8 activations: norm + quantise and SwiGLU + quantise happen inside the
        // GEMVs' staging phase (7 launches per layer).  The residual alternates between two
        // vectors because every CTA of a GEMV reads the old one while CTA 0 writes the new one.
        half* res_next = D->residual2;
        const size_t kvdim = (size_t)c.n_kv_heads * c.head_dim;
        for (int l = 0; l < c.n_layers; l++) {
            const LayerW& L = D->layers[l];
            const size_t kv_off = (size_t)l * kv_layer + kv_first;
            half *qb = D->qkv1, *kb = qb + qdim, *vb = kb + kvdim, *gb = D->gu1, *ub = gb + inter;
            if (l == 0) {
                TRY(launch_gemv_int8_packed_norm(L.qkv.p, res_cur, nullptr, L.attn_norm, nullptr, c.rms_norm_eps, qb,
                                                 L.qkv.rows, L.qkv.cols, s));
            } else {
                TRY(launch_gemv_int8_packed_norm(L.qkv.p, D->ffn_out, res_cur, L.attn_norm, res_next, c.rms_norm_eps, qb,
                                                 L.qkv.rows, L.qkv.cols, s));
                std::swap(res_cur, res_next);
            }
            TRY(launch_attention_decode(qb, kb, vb, D->k_cache + kv_off, D->v_cache + kv_off, D->attn_out, c.n_heads,
                                        c.n_kv_heads, c.head_dim, c.max_seq_len, start_pos, pos_dev, c.rope_theta,
                                        D->attn_ws2, D->attn_counters, s));
            TRY(launch_gemv_int8_packed_quant(L.o.p, D->attn_out, D->hidden2, L.o.rows, L.o.cols, s));
            TRY(launch_gemv_int8_packed_norm(L.gate_up.p, D->hidden2, res_cur, L.ffn_norm, res_next, c.rms_norm_eps, gb,
                                             L.gate_up.rows, L.gate_up.cols, s));
            std::swap(res_cur, res_next);
            TRY(launch_gemv_int8_packed_silu(L.down.p, gb, ub, D->ffn_out, L.down.rows, L.down.cols, s));
        }
    } else
    for (int l = 0; l < c.n_layers; l++) {
        const LayerW& L = D->layers[l];
        const size_t kv_off = (size_t)l * kv_layer + kv_first;
        // pre-attention norm; from the second layer on it also adds the previous FFN output
        if (l == 0)
            TRY(launch_rmsnorm(D->residual, L.attn_norm, D->hidden, nullptr, nullptr, xq, xs, n, hidden, c.rms_norm_eps, 0, s));
        else
            TRY(launch_rmsnorm(D->ffn_out, L.attn_norm, D->hidden, D->residual, D->residual, xq, xs, n, hidden,
                               c.rms_norm_eps, 1, s));
        half *qb = D->q, *kb = D->k, *vb = D->v, *gb = D->gate, *ub = D->up;
        if (n == 1 && L.qkv.p) {
            qb = D->qkv1;
            kb = qb + qdim;
            vb = kb + (size_t)c.n_kv_heads * c.head_dim;
            const PackedW* w[1] = {&L.qkv};
            half* y[1] = {qb};
            TRY(linear_multi(D, 1, w, y, D->hidden, i8, n, s));
        } else {
            const PackedW* w[3] = {&L.q, &L.k, &L.v};
            half* y[3] = {qb, kb, vb};
            TRY(linear_multi(D, 3, w, y, D->hidden, i8, n, s));
        }
        TRY(launch_rope(qb, kb, vb, D->k_cache + kv_off, D->v_cache + kv_off, bsz, seq_n, c.n_heads, c.n_kv_heads,
                        c.head_dim, start_pos, pos_dev, c.rope_theta, c.max_seq_len, 1, s));
        if (pos_dev)
            TRY(launch_attention(qb, D->k_cache + kv_off, D->v_cache + kv_off, D->attn_out, 1, c.n_heads, c.n_kv_heads,
                                 c.head_dim, 1, 1, c.max_seq_len, pos_dev, D->attn_ws, D->attn_counters, s));
        else
            TRY(launch_attention(qb, D->k_cache + kv_off, D->v_cache + kv_off, D->attn_out, bsz, c.n_heads, c.n_kv_heads,
                                 c.head_dim, seq_n, start_pos + seq_n, c.max_seq_len, nullptr, D->attn_ws, D->attn_counters, s));
        if (i8) TRY(launch_quantize_absmax_int8(D->attn_out, D->xq, D->xscale, qdim, s));
        {
            const PackedW* w[1] = {&L.o};
            half* y[1] = {D->hidden2};
            TRY(linear_multi(D, 1, w, y, D->attn_out, i8, n, s));
        }
        TRY(launch_rmsnorm(D->hidden2, L.ffn_norm, D->hidden, D->residual, D->residual, xq, xs, n, hidden, c.rms_norm_eps,
                           1, s));
        if (n == 1 && L.gate_up.p) {
            gb = D->gu1;
            ub = gb + inter;
            const PackedW* w[1] = {&L.gate_up};
            half* y[1] = {gb};
            TRY(linear_multi(D, 1, w, y, D->hidden, i8, n, s));
        } else {
            const PackedW* w[2] = {&L.gate, &L.up};
            half* y[2] = {gb, ub};
            TRY(linear_multi(D, 2, w, y, D->hidden, i8, n, s));
        }
        TRY(launch_silu_mul(gb, ub, gb, (long long)n * inter, xq, xs, s));
        {
            const PackedW* w[1] = {&L.down};
            half* y[1] = {D->ffn_out};
            TRY(linear_multi(D, 1, w, y, gb, i8, n, s));
        }
    }
    const bool tern_head = (c.lm_head_weight == nullptr);
    if (batch > 0) {
        // last residual add + final norm + lm_head for every sequence
        TRY(launch_rmsnorm(D->ffn_out, static_cast<const half*>(c.final_norm_weight), D->hidden, res_cur, res_cur, nullptr,
                           nullptr, n, hidden, c.rms_norm_eps, 1, s));
        if (tern_head) TRY(linear_f16(D->lm_head, D->hidden, D->logits, n, s));
        else TRY(launch_fp16_gemv_batched(static_cast<const half*>(c.lm_head_weight), D->hidden, D->logits, n, c.vocab_size, hidden, s));
        return TLLM_OK;
    }
    // last residual add + final norm, last token only
    const size_t last = (size_t)(n - 1) * hidden;
    const bool head_i8 = tern_head;     // a ternary lm_head always takes the INT8 path (src/transformer.cpp:308-311)
    half* logits = D->logits + (size_t)seq * c.vocab_size;
    TRY(launch_rmsnorm(D->ffn_out + last, static_cast<const half*>(c.final_norm_weight), D->hidden, res_cur + last,
                       res_cur + last, head_i8 ? D->xq : nullptr, head_i8 ? D->xscale : nullptr, 1, hidden,
                       c.rms_norm_eps, 1, s));
    if (tern_head) {
        const uint8_t* p[1] = {D->lm_head.p};
        half* y[1] = {logits};
        int rows[1] = {D->lm_head.rows};
        TRY(launch_gemv_int8_packed_multi(1, p, y, rows, D->lm_head.cols, D->xq, D->xscale, s));
    } else {
        TRY(launch_fp16_gemv(static_cast<const half*>(c.lm_head_weight), D->hidden, logits, c.vocab_size, hidden, s));
    }
#undef TRY
    return TLLM_OK;
}

}  // namespace

}  // namespace tllm

using namespace tllm;

extern "C" {

void tllm_b200_decoder_destroy(void* decoder)
{
    Decoder* D = static_cast<Decoder*>(decoder);
    if (!D) return;
    if (D->step_graph) cudaGraphExecDestroy(D->step_graph);
    if (D->stream) cudaStreamDestroy(D->stream);
    for (void* p : D->owned) cudaFree(p);
    delete D;
}

int tllm_b200_decoder_create(const tllm_b200_model_desc* desc, int flags, void** out)
{
    return tllm_b200_decoder_create_batched(desc, flags, 1, out);
}

int tllm_b200_decoder_create_batched(const tllm_b200_model_desc* desc, int flags, int max_batch, void** out)
{
    if (!desc || !out || !desc->layers || !desc->embedding_table || !desc->final_norm_weight)
        return fail(TLLM_ERR_NULL, "decoder_create: null argument");
    if (max_batch < 1 || max_batch > TLLM_DECODER_MAX_BATCH)
        return fail(TLLM_ERR_BATCH, "decoder_create: max_batch=%d outside 1..%d", max_batch, TLLM_DECODER_MAX_BATCH);
    const tllm_b200_model_desc& c = *desc;
    if (c.group_size != kGroup) return fail(TLLM_ERR_GROUP, "decoder_create: group_size=%d (must be 128)", c.group_size);
    if (c.n_layers <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.n_heads % c.n_kv_heads || c.head_dim % 8 ||
        c.hidden_dim % kGroup || c.intermediate_dim % kGroup || (c.n_heads * c.head_dim) % kGroup || c.max_seq_len <= 0)
        return fail(TLLM_ERR_SHAPE, "decoder_create: unsupported configuration");
    {
        // what the attention kernels take: head_dim 16/32/64/128, at most 16 query heads per KV head
        const int hd = c.head_dim, group = c.n_heads / c.n_kv_heads;
        if (!(hd == 16 || hd == 32 || hd == 64 || hd == 128) || group > 16 || group * (hd / 8) > 256)
            return fail(TLLM_ERR_SHAPE, "decoder_create: head_dim=%d with %d query heads per KV head is not supported", hd, group);
    }
    Decoder* D = new Decoder();
    D->d = c;
    D->flags = flags;
    D->max_batch = max_batch;
    int st = TLLM_OK;
    auto bail = [&](int code) {
        tllm_b200_decoder_destroy(D);
        return code;
    };
    if (cudaStreamCreateWithFlags(&D->stream, cudaStreamNonBlocking) != cudaSuccess)
        return bail(fail(TLLM_ERR_LAUNCH, "decoder_create: cudaStreamCreate failed"));
    D->layers.resize(c.n_layers);
    for (int l = 0; l < c.n_layers; l++) {
        const tllm_b200_layer_weights& w = c.layers[l];
        LayerW& L = D->layers[l];
        if (!w.attn_norm_weight || !w.ffn_norm_weight) return bail(fail(TLLM_ERR_NULL, "decoder_create: null norm weight"));
        L.attn_norm = static_cast<const half*>(w.attn_norm_weight);
        L.ffn_norm = static_cast<const half*>(w.ffn_norm_weight);
        {
            const tllm_b200_ternary_weight* src[3] = {&w.q_proj, &w.k_proj, &w.v_proj};
            PackedW* dst[3] = {&L.q, &L.k, &L.v};
            if ((st = pack_group(D, 3, src, dst, &L.qkv, D->stream))) return bail(st);
        }
        {
            const tllm_b200_ternary_weight* src[2] = {&w.gate_proj, &w.up_proj};
            PackedW* dst[2] = {&L.gate, &L.up};
            if ((st = pack_group(D, 2, src, dst, &L.gate_up, D->stream))) return bail(st);
        }
        if ((st = pack(D, w.o_proj, &L.o, D->stream)) || (st = pack(D, w.down_proj, &L.down, D->stream))) return bail(st);
    }
    D->fused_ok = true;
    for (const LayerW& L : D->layers) D->fused_ok = D->fused_ok && L.qkv.p && L.gate_up.p;
    D->d.layers = nullptr;      // the caller's array is not referenced after this call
    if (!c.lm_head_weight && (st = pack(D, c.lm_head_ternary, &D->lm_head, D->stream))) return bail(st);

    const size_t mt = (size_t)(c.max_seq_len > max_batch ? c.max_seq_len : max_batch);   // activation rows
    const size_t qdim = (size_t)c.n_heads * c.head_dim, kvdim = (size_t)c.n_kv_heads * c.head_dim;
    size_t maxdim = (size_t)c.hidden_dim > (size_t)c.intermediate_dim ? c.hidden_dim : c.intermediate_dim;
    if (qdim > maxdim) maxdim = qdim;
    const size_t kv_elems = (size_t)c.n_layers * max_batch * c.max_seq_len * kvdim;
#define ALLOC(x) do { if ((st = (x)) != TLLM_OK) return bail(st); } while (0)
    ALLOC(dev_alloc(D, &D->residual, mt * c.hidden_dim, true));
    ALLOC(dev_alloc(D, &D->hidden, mt * c.hidden_dim, true));
    ALLOC(dev_alloc(D, &D->hidden2, mt * c.hidden_dim, true));
    ALLOC(dev_alloc(D, &D->q, mt * qdim, true));
    ALLOC(dev_alloc(D, &D->k, mt * kvdim, true));
    ALLOC(dev_alloc(D, &D->v, mt * kvdim, true));
    ALLOC(dev_alloc(D, &D->attn_out, mt * qdim, true));
    ALLOC(dev_alloc(D, &D->gate, mt * c.intermediate_dim, true));
    ALLOC(dev_alloc(D, &D->up, mt * c.intermediate_dim, true));
    ALLOC(dev_alloc(D, &D->ffn_out, mt * c.hidden_dim, true));
    ALLOC(dev_alloc(D, &D->logits, (size_t)max_batch * c.vocab_size, true));
    ALLOC(dev_alloc(D, &D->k_cache, kv_elems, true));
    ALLOC(dev_alloc(D, &D->v_cache, kv_elems, true));
    ALLOC(dev_alloc(D, &D->residual2, (size_t)c.hidden_dim, true));
    ALLOC(dev_alloc(D, &D->qkv1, qdim + 2 * kvdim, true));
    ALLOC(dev_alloc(D, &D->gu1, (size_t)2 * c.intermediate_dim, true));
    ALLOC(dev_alloc(D, &D->xq, maxdim, true));
    ALLOC(dev_alloc(D, &D->xscale, 4, true));
    ALLOC(dev_alloc(D, &D->attn_ws, attention_workspace_bytes(max_batch, c.n_heads, c.n_kv_heads, c.head_dim, c.max_seq_len) / sizeof(float), true));
    ALLOC(dev_alloc(D, &D->attn_ws2, attention_decode_workspace_bytes(c.n_heads, c.n_kv_heads, c.head_dim, c.max_seq_len) / sizeof(float), true));
    ALLOC(dev_alloc(D, &D->attn_counters, (size_t)max_batch * c.n_kv_heads, true));
    ALLOC(dev_alloc(D, &D->state, 4, true));
    D->history_cap = c.max_seq_len;
    ALLOC(dev_alloc(D, &D->history, (size_t)D->history_cap, true));
    ALLOC(dev_alloc(D, &D->am_val, 64, true));
    ALLOC(dev_alloc(D, &D->am_idx, 64, true));
    ALLOC(dev_alloc(D, &D->am_counter, 1, true));
#undef ALLOC
    if (cudaStreamSynchronize(D->stream) != cudaSuccess)
        return bail(fail(TLLM_ERR_LAUNCH, "decoder_create: %s", cudaGetErrorString(cudaGetLastError())));
    *out = D;
    return TLLM_OK;
}

int tllm_b200_decoder_reset(void* decoder, void* stream)
{
    Decoder* D = static_cast<Decoder*>(decoder);
    if (!D) return fail(TLLM_ERR_NULL, "decoder_reset: null decoder");
    const size_t bytes = (size_t)D->d.n_layers * D->max_batch * D->d.max_seq_len * D->d.n_kv_heads * D->d.head_dim * sizeof(half);
    cudaMemsetAsync(D->k_cache, 0, bytes, static_cast<cudaStream_t>(stream));
    cudaMemsetAsync(D->v_cache, 0, bytes, static_cast<cudaStream_t>(stream));
    return check_launch("decoder_reset");
}

int tllm_b200_decoder_forward(void* decoder, const int* token_ids, int n_tokens, int start_pos, void** logits,
                              void* stream)
{
    return tllm_b200_decoder_forward_seq(decoder, 0, token_ids, n_tokens, start_pos, logits, stream);
}

int tllm_b200_decoder_forward_seq(void* decoder, int seq, const int* token_ids, int n_tokens, int start_pos,
                                  void** logits, void* stream)
{
    Decoder* D = static_cast<Decoder*>(decoder);
    if (!D || !token_ids || !logits) return fail(TLLM_ERR_NULL, "decoder_forward: null argument");
    if (seq < 0 || seq >= D->max_batch) return fail(TLLM_ERR_BATCH, "decoder_forward: sequence %d outside 0..%d", seq, D->max_batch - 1);
    if (n_tokens < 1 || start_pos < 0 || start_pos + n_tokens > D->d.max_seq_len)
        return fail(TLLM_ERR_SHAPE, "decoder_forward: n_tokens=%d start_pos=%d max_seq_len=%d", n_tokens, start_pos,
                    D->d.max_seq_len);
    const int st = forward(D, token_ids, n_tokens, start_pos, nullptr, seq, 0, static_cast<cudaStream_t>(stream));
    if (st) return st;
    *logits = D->logits + (size_t)seq * D->d.vocab_size;
    return TLLM_OK;
}

int tllm_b200_decoder_forward_batch(void* decoder, const int* token_ids, int batch, int pos, void** logits, void* stream)
{
    Decoder* D = static_cast<Decoder*>(decoder);
    if (!D || !token_ids || !logits) return fail(TLLM_ERR_NULL, "decoder_forward_batch: null argument");
    if (batch < 1 || batch > D->max_batch) return fail(TLLM_ERR_BATCH, "decoder_forward_batch: batch=%d outside 1..%d", batch, D->max_batch);
    if (pos < 0 || pos >= D->d.max_seq_len) return fail(TLLM_ERR_SHAPE, "decoder_forward_batch: pos=%d max_seq_len=%d", pos, D->d.max_seq_len);
    const int st = forward(D, token_ids, batch, pos, nullptr, 0, batch, static_cast<cudaStream_t>(stream));
    if (st) return st;
    *logits = D->logits;
    return TLLM_OK;
}

int tllm_b200_decoder_generate(void* decoder, int first_token, int start_pos, int n_steps, int* tokens_host,
                               float* ms_per_step_host)
{
    Decoder* D = static_cast<Decoder*>(decoder);
    if (!D || !tokens_host) return fail(TLLM_ERR_NULL, "decoder_generate: null argument");
    if (n_steps < 1 || n_steps > D->history_cap || start_pos < 0 || start_pos + n_steps > D->d.max_seq_len)
        return fail(TLLM_ERR_SHAPE, "decoder_generate: n_steps=%d start_pos=%d max_seq_len=%d", n_steps, start_pos,
                    D->d.max_seq_len);
    cudaStream_t s = D->stream;
    int st;
    // work queued by the caller on other streams (a prefill) must be complete
    if (cudaDeviceSynchronize() != cudaSuccess) return fail(TLLM_ERR_LAUNCH, "decoder_generate: %s", cudaGetErrorString(cudaGetLastError()));
    const int init[3] = {first_token, start_pos, 0};
    cudaMemcpyAsync(D->state, init, sizeof(init), cudaMemcpyHostToDevice, s);
    auto step = [&]() -> int {
        int e = forward(D, D->state, 1, 0, D->state + 1, 0, 0, s);
        if (e) return e;
        return launch_argmax(D->logits, D->d.vocab_size, D->state, D->history, D->state + 2, D->am_val, D->am_idx,
                             D->am_counter, D->state + 1, s);
    };
    if (!D->step_graph) {
        // One eager step first: it performs every lazy set-up (scratch allocation, kernel
        // attributes) outside the capture.  A step rewrites the same cache slot and
        // buffers when repeated, so the state is put back and the step captured.
        if ((st = step())) return st;
        if (cudaStreamSynchronize(s) != cudaSuccess) return fail(TLLM_ERR_LAUNCH, "decoder_generate: %s", cudaGetErrorString(cudaGetLastError()));
        cudaMemcpyAsync(D->state, init, sizeof(init), cudaMemcpyHostToDevice, s);
        cudaGraph_t g = nullptr;
        if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) != cudaSuccess)
            return fail(TLLM_ERR_LAUNCH, "decoder_generate: begin capture: %s", cudaGetErrorString(cudaGetLastError()));
        st = step();
        const cudaError_t ce = cudaStreamEndCapture(s, &g);
        if (st) {
            if (g) cudaGraphDestroy(g);
            return st;
        }
        if (ce != cudaSuccess || !g) return fail(TLLM_ERR_LAUNCH, "decoder_generate: end capture: %s", cudaGetErrorString(cudaGetLastError()));
        const cudaError_t ie = cudaGraphInstantiate(&D->step_graph, g, 0);
        cudaGraphDestroy(g);
        if (ie != cudaSuccess) return fail(TLLM_ERR_LAUNCH, "decoder_generate: instantiate: %s", cudaGetErrorString(cudaGetLastError()));
    }
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, s);
    for (int i = 0; i < n_steps; i++) {
        if (cudaGraphLaunch(D->step_graph, s) != cudaSuccess) {
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
            return fail(TLLM_ERR_LAUNCH, "decoder_generate: graph launch: %s", cudaGetErrorString(cudaGetLastError()));
        }
    }
    cudaEventRecord(e1, s);
    cudaMemcpyAsync(tokens_host, D->history, sizeof(int) * n_steps, cudaMemcpyDeviceToHost, s);
    const cudaError_t se = cudaStreamSynchronize(s);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (se != cudaSuccess) return fail(TLLM_ERR_LAUNCH, "decoder_generate: %s", cudaGetErrorString(se));
    if (ms_per_step_host) *ms_per_step_host = ms / (float)n_steps;
    return device_error_check(s);
}

}  // extern "C"
