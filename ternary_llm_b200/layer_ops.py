"""Host-side mirror of the reference's layer operators (its include/kernels.cuh:45-84,
namespace ternary): same names, argument order and meaning, calling the C ABI of
include/tllm_b200_layer.h with the tensors' device pointers on torch's current stream.
PyTorch only owns the memory; nothing here computes on the CPU or with torch ops.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .ops import PreparedWeight, _chk, _stream

_H = torch.float16


def rmsnorm_forward(input, weight, output, residual, residual_out, batch: int, dim: int, eps: float) -> None:
    """output = rmsnorm(input (+ residual)) * weight; the sum goes to residual_out when given
    (reference include/kernels.cuh:45-48)."""
    _lib.check(_lib.lib().tllm_b200_rmsnorm(
        _chk(input, _H, "input"), _chk(weight, _H, "weight"), _chk(output, _H, "output"),
        _chk(residual, _H, "residual") if residual is not None else None,
        _chk(residual_out, _H, "residual_out") if residual_out is not None else None,
        batch, dim, eps, _stream()))


def rope_forward(q, k, batch: int, seq_len: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 start_pos: int, theta: float) -> None:
    """In-place rotary embedding on q and k (reference include/kernels.cuh:50-53)."""
    _lib.check(_lib.lib().tllm_b200_rope(_chk(q, _H, "q"), _chk(k, _H, "k"), batch, seq_len, n_heads,
                                         n_kv_heads, head_dim, start_pos, theta, _stream()))


def copy_to_kv_cache(k, v, k_cache, v_cache, batch: int, n_kv_heads: int, head_dim: int, seq_len: int,
                     start_pos: int, max_seq_len: int) -> None:
    """Appends k, v at cache positions start_pos.. (reference include/kernels.cuh:72-76)."""
    _lib.check(_lib.lib().tllm_b200_copy_to_kv_cache(
        _chk(k, _H, "k"), _chk(v, _H, "v"), _chk(k_cache, _H, "k_cache"), _chk(v_cache, _H, "v_cache"),
        batch, n_kv_heads, head_dim, seq_len, start_pos, max_seq_len, _stream()))


def rope_append(q, k, v, k_cache, v_cache, batch: int, seq_len: int, n_heads: int, n_kv_heads: int,
                head_dim: int, start_pos: int, theta: float, max_seq_len: int) -> None:
    """rope_forward and copy_to_kv_cache in one launch."""
    _lib.check(_lib.lib().tllm_b200_rope_append(
        _chk(q, _H, "q"), _chk(k, _H, "k"), _chk(v, _H, "v"), _chk(k_cache, _H, "k_cache"),
        _chk(v_cache, _H, "v_cache"), batch, seq_len, n_heads, n_kv_heads, head_dim, start_pos, theta,
        max_seq_len, _stream()))


def attention_forward(q, k_cache, v_cache, output, batch: int, n_heads: int, n_kv_heads: int, head_dim: int,
                      seq_len: int, kv_len: int, kv_len_max: int) -> None:
    """Causal grouped-query attention over the KV cache (reference include/kernels.cuh:55-58)."""
    _lib.check(_lib.lib().tllm_b200_attention(
        _chk(q, _H, "q"), _chk(k_cache, _H, "k_cache"), _chk(v_cache, _H, "v_cache"), _chk(output, _H, "output"),
        batch, n_heads, n_kv_heads, head_dim, seq_len, kv_len, kv_len_max, _stream()))


def attention_decode(q, k, v, k_cache, v_cache, output, n_heads: int, n_kv_heads: int, head_dim: int, pos: int,
                     theta: float, max_seq_len: int) -> None:
    """One new token of one sequence: rotary embedding, cache append and attention over
    positions 0..pos in one launch (rope_forward + copy_to_kv_cache + attention_forward)."""
    _lib.check(_lib.lib().tllm_b200_attention_decode(
        _chk(q, _H, "q", n_heads * head_dim), _chk(k, _H, "k", n_kv_heads * head_dim), _chk(v, _H, "v", n_kv_heads * head_dim),
        _chk(k_cache, _H, "k_cache", n_kv_heads * max_seq_len * head_dim),
        _chk(v_cache, _H, "v_cache", n_kv_heads * max_seq_len * head_dim), _chk(output, _H, "output", n_heads * head_dim),
        n_heads, n_kv_heads, head_dim, pos, theta, max_seq_len, _stream()))


def silu_mul_forward(gate, up, output, size: int) -> None:
    """output = silu(gate) * up (reference include/kernels.cuh:60-62)."""
    _lib.check(_lib.lib().tllm_b200_silu_mul(_chk(gate, _H, "gate"), _chk(up, _H, "up"),
                                             _chk(output, _H, "output"), size, _stream()))


def add_forward(a, b, output, size: int) -> None:
    """output = a + b (reference include/kernels.cuh:64-66)."""
    _lib.check(_lib.lib().tllm_b200_add(_chk(a, _H, "a"), _chk(b, _H, "b"), _chk(output, _H, "output"),
                                        size, _stream()))


def embedding_lookup(table, indices, output, n_tokens: int, dim: int) -> None:
    """output[t] = table[indices[t]] (reference include/kernels.cuh:68-70)."""
    _lib.check(_lib.lib().tllm_b200_embedding_lookup(_chk(table, _H, "table"), _chk(indices, torch.int32, "indices"),
                                                     _chk(output, _H, "output"), n_tokens, dim, _stream()))


def fp16_gemv(weight, input, output, rows: int, cols: int) -> None:
    """output = weight @ input in FP16 with FP32 accumulation (reference include/kernels.cuh:78-80)."""
    _lib.check(_lib.lib().tllm_b200_fp16_gemv(_chk(weight, _H, "weight"), _chk(input, _H, "input"),
                                              _chk(output, _H, "output"), rows, cols, _stream()))


def fp16_gemm(A, B, C, M: int, N: int, K: int) -> None:
    """C[M,N] = A[M,K] @ B[N,K]^T (reference include/kernels.cuh:82-84)."""
    _lib.check(_lib.lib().tllm_b200_fp16_gemm(_chk(A, _H, "A"), _chk(B, _H, "B"), _chk(C, _H, "C"), M, N, K,
                                              _stream()))


def ternary_gemv_int8_packed_multi(weights, input_int8, input_scale_dev, outputs) -> None:
    """INT8 GEMV over 1..4 prepared matrices sharing the quantised vector; the activation
    scale is the device float the quantiser wrote (no host read in between)."""
    n = len(weights)
    cols = weights[0].cols
    packed = (ctypes.c_void_p * n)(*[w.packed.data_ptr() for w in weights])
    ys = (ctypes.c_void_p * n)(*[_chk(y, _H, "output") for y in outputs])
    rows = (ctypes.c_int * n)(*[w.rows for w in weights])
    _lib.check(_lib.lib().tllm_b200_gemv_int8_packed_multi(
        n, packed, ys, rows, cols, _chk(input_int8, torch.int8, "input_int8"),
        _chk(input_scale_dev, torch.float32, "input_scale_dev"), _stream()))
