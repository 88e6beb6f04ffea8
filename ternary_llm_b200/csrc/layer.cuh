// Launchers of the layer operators (layer_ops.cu, attention.cu), shared with the C ABI
// and the decoder.
#pragma once
#include "common.cuh"

namespace tllm {

// q / q_scale: when not null the normalised vector is also quantised (one scale per row).
// round_first: the variance is taken over the FP16-rounded sum (what a separate
// add-then-normalise sequence computes) instead of the unrounded one.
int launch_rmsnorm(const half* input, const half* weight, half* output, const half* residual, half* residual_out,
                   int8_t* q, float* q_scale, int batch, int dim, float eps, int round_first, cudaStream_t stream);
// pos_dev: start_pos is read from device memory when not null.  Caches may be null (rotation
// only); do_rope == 0 appends without rotating.
int launch_rope(half* q, half* k, const half* v, half* k_cache, half* v_cache, int batch, int seq_len, int n_heads,
                int n_kv_heads, int head_dim, int start_pos, const int* pos_dev, float theta, int max_seq_len,
                int do_rope, cudaStream_t stream);
// q / q_scale not null: one vector, output also quantised.
int launch_silu_mul(const half* gate, const half* up, half* out, long long size, int8_t* q, float* q_scale,
                    cudaStream_t stream);
int launch_add(const half* a, const half* b, half* out, long long size, cudaStream_t stream);
int launch_embedding(const half* table, const int* indices, half* out, int n_tokens, int dim, cudaStream_t stream);
int launch_fp16_gemv(const half* w, const half* x, half* y, int rows, int cols, cudaStream_t stream);
// y[b, r] = W[r, :] . x[b, :] for `batch` vectors (x [batch, cols], y [batch, rows]).
int launch_fp16_gemv_batched(const half* w, const half* x, half* y, int batch, int rows, int cols, cudaStream_t stream);
int launch_fp16_gemm(const half* A, const half* B, half* C, int M, int N, int K, cudaStream_t stream);
// part_val / part_idx: 64 entries each; counter: one zero-initialised unsigned; pos: when not
// null, *pos is advanced by one together with the token (the decode loop's cache position).
int launch_argmax(const half* logits, int n, int* out, int* history, int* step, float* part_val, int* part_idx,
                  unsigned* counter, int* pos, cudaStream_t stream);

size_t attention_workspace_bytes(int batch, int n_heads, int n_kv_heads, int head_dim, int kv_len_max);
// kv_len_dev: decode only, kv_len = kv_len + *kv_len_dev.  ws / counters: decode split scratch or null.
int launch_attention(const half* q, const half* k_cache, const half* v_cache, half* out, int batch, int n_heads,
                     int n_kv_heads, int head_dim, int seq_len, int kv_len, int kv_len_max, const int* kv_len_dev,
                     float* ws, unsigned* counters, cudaStream_t stream);

// Single-token step: RoPE + cache append + attention in one launch (q is read unrotated and not
// modified; the rotated key and the value go to cache position pos, or *pos_dev).
size_t attention_decode_workspace_bytes(int n_heads, int n_kv_heads, int head_dim, int kv_len_max);
int launch_attention_decode(half* q, const half* k, const half* v, half* k_cache, half* v_cache, half* out, int n_heads,
                            int n_kv_heads, int head_dim, int kv_len_max, int pos, const int* pos_dev, float theta,
                            float* ws, unsigned* counters, cudaStream_t stream);

}  // namespace tllm
