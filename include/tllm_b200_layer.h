/*
 * tllm_b200_layer.h -- the operators either side of the ternary contraction inside a
 * decoder layer, and a decoder that runs the reference engine's forward pass with them.
 *
 * The reference engine (jastaq/ternary-llm) declares these operators beside the ternary
 * contraction in its include/kernels.cuh:45-86 and calls them from
 * Transformer::forward (src/transformer.cpp:168-318).  Each function below cites the
 * declaration it replaces; argument meaning and tensor layouts are the reference's:
 *
 *   activations   half [batch, seq_len, heads, head_dim] / [tokens, dim], row-major
 *   KV caches     half [batch, n_kv_heads, max_seq_len, head_dim]
 *
 * All pointers are device pointers unless a name ends in _host; `stream` is a
 * cudaStream_t passed as void*.  Functions return TLLM_OK or a negative status of
 * tllm_b200.h.  Nothing here falls back to a CPU path.
 */
#ifndef TLLM_B200_LAYER_H
#define TLLM_B200_LAYER_H

#include "tllm_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- stand-alone operators (reference interface, one call each) ---------------- */

/* rmsnorm_forward, include/kernels.cuh:45-48 (kernels/rmsnorm.cu).  tmp = input (+
 * residual when not NULL; the sum is stored to residual_out when not NULL);
 * output = tmp * rsqrt(mean(tmp^2) + eps) * weight.  One vector of `dim` per batch row. */
int tllm_b200_rmsnorm(const void* input, const void* weight, void* output, const void* residual,
                      void* residual_out, int batch, int dim, float eps, void* stream);

/* rope_forward, include/kernels.cuh:50-53 (kernels/rope.cu): in place on q and k,
 * interleaved pairs (2i, 2i+1), angle = (start_pos + s) / theta^(2i/head_dim). */
int tllm_b200_rope(void* q, void* k, int batch, int seq_len, int n_heads, int n_kv_heads, int head_dim,
                   int start_pos, float theta, void* stream);

/* copy_to_kv_cache, include/kernels.cuh:72-76 (kernels/elementwise.cu:97-147). */
int tllm_b200_copy_to_kv_cache(const void* k, const void* v, void* k_cache, void* v_cache, int batch,
                               int n_kv_heads, int head_dim, int seq_len, int start_pos, int max_seq_len,
                               void* stream);

/* Both of the above in one launch: rotate q and k in place and append the rotated k
 * and v at cache position start_pos + s.  No counterpart in the reference (it makes two
 * launches, src/transformer.cpp:225-236). */
int tllm_b200_rope_append(void* q, void* k, const void* v, void* k_cache, void* v_cache, int batch, int seq_len,
                          int n_heads, int n_kv_heads, int head_dim, int start_pos, float theta,
                          int max_seq_len, void* stream);

/* attention_forward, include/kernels.cuh:55-58 (kernels/attention.cu): causal softmax
 * attention with grouped-query heads; query s of the call sits at position
 * kv_len - seq_len + s.  Every seq_len computes the softmax that the reference documents
 * (its multi-token kernel does not: see csrc/attention.cu).  A single-token call over a
 * cache of more than 256 positions is split over the cache positions; the partial results
 * go through a per-device scratch buffer that this call allocates (and grows) on demand --
 * so the first call with given sizes must not happen during stream capture
 * (TLLM_ERR_LAUNCH), and calls of one device must be issued in stream order. */
int tllm_b200_attention(const void* q, const void* k_cache, const void* v_cache, void* output, int batch,
                        int n_heads, int n_kv_heads, int head_dim, int seq_len, int kv_len, int kv_len_max,
                        void* stream);

/* One new token of one sequence: rope_forward on q and k, copy_to_kv_cache of the rotated k
 * and v at position pos, and attention_forward over positions 0..pos, in ONE launch whose
 * CTAs each own 64 cache positions of a KV head.  q [n_heads, head_dim] is rotated in place;
 * k, v [n_kv_heads, head_dim] as the projections wrote them; caches [n_kv_heads, max_seq_len,
 * head_dim].  No counterpart in the reference (it makes three launches,
 * src/transformer.cpp:225-245).  Uses the same per-device scratch as tllm_b200_attention:
 * the first call with given sizes must not happen during stream capture. */
int tllm_b200_attention_decode(void* q, const void* k, const void* v, void* k_cache, void* v_cache, void* output,
                               int n_heads, int n_kv_heads, int head_dim, int pos, float theta, int max_seq_len,
                               void* stream);

/* silu_mul_forward, include/kernels.cuh:60-62 (kernels/activations.cu:18-74). */
int tllm_b200_silu_mul(const void* gate, const void* up, void* output, int size, void* stream);

/* add_forward, include/kernels.cuh:64-66 (kernels/elementwise.cu:19-49). */
int tllm_b200_add(const void* a, const void* b, void* output, int size, void* stream);

/* embedding_lookup, include/kernels.cuh:68-70 (kernels/elementwise.cu:55-88). */
int tllm_b200_embedding_lookup(const void* table, const int* indices, void* output, int n_tokens, int dim,
                               void* stream);

/* fp16_gemv, include/kernels.cuh:78-80 (kernels/elementwise.cu:158-201): the FP16 lm_head. */
int tllm_b200_fp16_gemv(const void* weight, const void* input, void* output, int rows, int cols, void* stream);

/* fp16_gemm, include/kernels.cuh:82-84 (kernels/elementwise.cu:216-304): C = A . B^T. */
int tllm_b200_fp16_gemm(const void* A, const void* B, void* C, int M, int N, int K, void* stream);

/* INT8 GEMV over up to TLLM_MAX_FUSED prepared matrices that share the quantised
 * activation vector, with the activation scale read from device memory (the float the
 * quantiser wrote), so that no host read sits between quantiser and GEMV as it does in
 * the reference (src/transformer.cpp:132-136,201-203,266-268).  No counterpart there. */
int tllm_b200_gemv_int8_packed_multi(int count, const void* const* packed, void* const* y, const int* rows,
                                     int cols, const void* x_int8, const float* input_scale_dev, void* stream);

/* ---- decoder: the reference's Transformer on these operators -------------------- */

/* TernaryWeight, include/model.h:17-36. */
typedef struct tllm_b200_ternary_weight {
    const void* nonzero_masks; /* uint32 [out_features, in_features/32] */
    const void* sign_masks;    /* uint32 [out_features, in_features/32] */
    const void* scales;        /* half   [out_features, in_features/group_size] */
    int out_features;
    int in_features;
} tllm_b200_ternary_weight;

/* TransformerLayer, include/model.h:41-56. */
typedef struct tllm_b200_layer_weights {
    tllm_b200_ternary_weight q_proj, k_proj, v_proj, o_proj, gate_proj, up_proj, down_proj;
    const void* attn_norm_weight; /* half [hidden_dim] */
    const void* ffn_norm_weight;  /* half [hidden_dim] */
} tllm_b200_layer_weights;

/* ModelConfig (include/config.h:11-30) and the Model's tensors (include/model.h:61-84). */
typedef struct tllm_b200_model_desc {
    int vocab_size, hidden_dim, intermediate_dim, n_layers, n_heads, n_kv_heads, max_seq_len, head_dim;
    int group_size;
    float rope_theta, rms_norm_eps;
    const void* embedding_table;   /* half [vocab, hidden] */
    const void* final_norm_weight; /* half [hidden] */
    const void* lm_head_weight;    /* half [vocab, hidden], or NULL when the lm_head is ternary */
    tllm_b200_ternary_weight lm_head_ternary;
    const tllm_b200_layer_weights* layers; /* host array of n_layers */
} tllm_b200_model_desc;

#define TLLM_DECODER_MAX_BATCH 64
#define TLLM_DECODER_INT8_DECODE 1 /* single-token steps quantise activations to INT8 (the reference's choice, src/transformer.cpp:182) */

/* Transformer::Transformer, src/transformer.cpp:29-72: allocates the KV caches and the
 * activation buffers, and repacks every ternary matrix of the model (a second copy of
 * the weights, 2.125 bits each; the caller's arrays are not referenced afterwards except
 * embedding, norms and an FP16 lm_head).  *out receives the handle. */
int tllm_b200_decoder_create(const tllm_b200_model_desc* desc, int flags, void** out);
void tllm_b200_decoder_destroy(void* decoder);

/* The same with room for max_batch (1..TLLM_DECODER_MAX_BATCH) independent sequences, each
 * with its own KV cache.  The reference's Transformer serves one sequence
 * (src/transformer.cpp:226-242 pass batch 1 to every operator although the operators take a
 * batch); no counterpart there. */
int tllm_b200_decoder_create_batched(const tllm_b200_model_desc* desc, int flags, int max_batch, void** out);

/* Transformer::reset, src/transformer.cpp:91-97. */
int tllm_b200_decoder_reset(void* decoder, void* stream);

/* Transformer::forward, src/transformer.cpp:168-318: embeds n_tokens token ids, runs the
 * layer stack with the cache positions start_pos.., and returns in *logits a device
 * pointer to half [vocab] for the last token (owned by the decoder). */
int tllm_b200_decoder_forward(void* decoder, const int* token_ids, int n_tokens, int start_pos, void** logits,
                              void* stream);

/* forward for sequence `seq` (0..max_batch-1) of a batched decoder: its own KV cache, logits
 * in its own row of the decoder's [max_batch, vocab] buffer. */
int tllm_b200_decoder_forward_seq(void* decoder, int seq, const int* token_ids, int n_tokens, int start_pos,
                                  void** logits, void* stream);

/* One decode step of `batch` sequences in lock step: token_ids[b] is the next token of
 * sequence b, all at cache position pos; the weights are read once for the whole batch (FP16
 * activations: passes of the streaming GEMV up to 6 sequences, the tcgen05 GEMM above).
 * *logits: half [batch, vocab]. */
int tllm_b200_decoder_forward_batch(void* decoder, const int* token_ids, int batch, int pos, void** logits,
                                    void* stream);

/* The greedy decode loop of the reference's generate() (src/main.cpp:140-163, sampling
 * reduced to argmax) with nothing on the host inside it: one decode step -- forward of
 * one token, argmax on the device, position advance -- is captured as a CUDA graph and
 * replayed n_steps times; the token, the position and the activation scales stay in
 * device memory.  tokens_host receives the n_steps generated tokens; the call returns
 * after they arrived.  first_token sits at position start_pos. */
int tllm_b200_decoder_generate(void* decoder, int first_token, int start_pos, int n_steps, int* tokens_host,
                               float* ms_per_step_host);

#ifdef __cplusplus
}
#endif
#endif /* TLLM_B200_LAYER_H */
