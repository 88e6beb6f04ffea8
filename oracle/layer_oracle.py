"""CPU restatement (numpy) of the reference's layer operators and of its forward pass.

TEST INFRASTRUCTURE ONLY: imported by tests/ (and nothing in the shipped package).
Each function follows the reference kernel it cites: FP16 tensors in and out, FP32
arithmetic inside, rounding to FP16 where the reference stores FP16.  Reduction order
is numpy's, not the kernels', so comparisons carry a tolerance stated in the tests.

Pinning: the reference ships no golden vectors for these operators.  On a machine with a
GPU the tests compare this restatement -- and the library -- with the reference's own
kernels compiled from its sources (oracle/_ref/libref.so).  Its multi-token attention
kernel does not compute a softmax (kernels/attention.cu:230-296 normalise by a
per-thread partial sum), so multi-token attention is checked against this restatement of
the documented operator only: parity unpinned for that one case.
"""
from __future__ import annotations

import numpy as np

from . import oracle as O

f32, f16 = np.float32, np.float16


def rmsnorm(x, weight, eps, residual=None, store_residual=True, round_first=False):
    """kernels/rmsnorm.cu:19-103.  x [batch, dim] FP16.  Returns (out, residual_out)."""
    v = x.astype(f32)
    res_out = None
    if residual is not None:
        v = v + residual.astype(f32)
        unrounded = v
        if store_residual:
            res_out = v.astype(f16)
            v = res_out.astype(f32)
        ss_src = v if round_first else unrounded
    else:
        ss_src = v
    var = (ss_src.astype(f32) ** 2).sum(axis=-1, dtype=f32, keepdims=True) / f32(x.shape[-1])
    rinv = f32(1.0) / np.sqrt(var + f32(eps), dtype=f32)
    out = (v * rinv * weight.astype(f32)).astype(f16)
    return out, res_out


def rope(x, start_pos, theta):
    """kernels/rope.cu:21-78.  x [batch, seq, heads, head_dim] FP16; interleaved pairs."""
    b, s, h, d = x.shape
    i = np.arange(d // 2, dtype=f32)
    freq = f32(1.0) / np.power(f32(theta), (f32(2.0) * i) / f32(d), dtype=f32)
    pos = (start_pos + np.arange(s)).astype(f32)
    ang = (pos[:, None] * freq[None, :]).astype(f32).astype(np.float64)
    cs, sn = np.cos(ang).astype(f32), np.sin(ang).astype(f32)
    x0 = x[..., 0::2].astype(f32)
    x1 = x[..., 1::2].astype(f32)
    out = np.empty_like(x)
    out[..., 0::2] = (x0 * cs[None, :, None, :] - x1 * sn[None, :, None, :]).astype(f16)
    out[..., 1::2] = (x0 * sn[None, :, None, :] + x1 * cs[None, :, None, :]).astype(f16)
    return out


def copy_to_kv_cache(k, v, k_cache, v_cache, start_pos):
    """kernels/elementwise.cu:97-128.  k, v [batch, seq, kv_heads, hd]; caches
    [batch, kv_heads, max_seq, hd], modified in place; positions past the end dropped."""
    b, s, h, d = k.shape
    max_seq = k_cache.shape[2]
    for t in range(s):
        p = start_pos + t
        if p < max_seq:
            k_cache[:, :, p, :] = k[:, t]
            v_cache[:, :, p, :] = v[:, t]


def attention(q, k_cache, v_cache, kv_len):
    """The operator documented at kernels/attention.cu:1-12 and computed by its decode
    kernel (:30-166): q [batch, seq, heads, hd]; query s sits at position kv_len - seq + s
    and sees cache positions up to its own; softmax(q.k / sqrt(hd)) . v in FP32."""
    b, s, h, d = q.shape
    hk = k_cache.shape[1]
    g = h // hk
    out = np.empty_like(q)
    scale = f32(1.0) / np.sqrt(f32(d))
    for bi in range(b):
        for hi in range(h):
            kc = k_cache[bi, hi // g].astype(f32)
            vc = v_cache[bi, hi // g].astype(f32)
            for si in range(s):
                lim = kv_len - s + si + 1
                sc = (kc[:lim] @ q[bi, si, hi].astype(f32)) * scale
                p = np.exp(sc - sc.max(), dtype=f32)
                p = p / p.sum(dtype=f32)
                out[bi, si, hi] = (p @ vc[:lim]).astype(f16)
    return out


def silu_mul(gate, up):
    """kernels/activations.cu:18-60."""
    g, u = gate.astype(f32), up.astype(f32)
    return (g / (f32(1.0) + np.exp(-g, dtype=f32)) * u).astype(f16)


def add(a, b):
    """kernels/elementwise.cu:19-36."""
    return (a.astype(f32) + b.astype(f32)).astype(f16)


def embedding_lookup(table, indices):
    """kernels/elementwise.cu:55-75."""
    return table[np.asarray(indices)]


def fp16_gemv(w, x):
    """kernels/elementwise.cu:158-188: FP32 accumulation, FP16 result."""
    return (w.astype(f32) @ x.astype(f32)).astype(f16)


def fp16_gemm(a, b):
    """kernels/elementwise.cu:216-289: C = A . B^T."""
    return (a.astype(f32) @ b.astype(f32).T).astype(f16)


class Transformer:
    """src/transformer.cpp:168-318 on the functions above: FP16 activations through
    ternary_gemm for several tokens, INT8-quantised activations through ternary_gemv_int8
    for one token (int8_decode), residual adds as separate FP16-rounded steps."""

    def __init__(self, model, int8_decode=True):
        self.m, self.c = model, model.config
        self.int8 = int8_decode
        c = self.c
        shape = (c.n_layers, 1, c.n_kv_heads, c.max_seq_len, c.head_dim)
        self.k_cache = np.zeros(shape, f16)
        self.v_cache = np.zeros(shape, f16)

    def _linear(self, t, x, int8):
        if int8:
            q, scale = O.quantize_absmax_int8(x[0])
            return O.ternary_matvec_int8(t.nonzero_masks, t.sign_masks, t.scales, q, scale).astype(f16)[None, :]
        return O.ternary_gemm(x, t.nonzero_masks, t.sign_masks, t.scales).astype(f16)

    def forward(self, tokens, start_pos):
        c, m = self.c, self.m
        n = len(tokens)
        i8 = self.int8 and n == 1
        res = embedding_lookup(m.embedding, tokens)
        for li, L in enumerate(m.layers):
            h, _ = rmsnorm(res, L["attn_norm"], c.rms_norm_eps)
            q = self._linear(L["q_proj"], h, i8).reshape(1, n, c.n_heads, c.head_dim)
            k = self._linear(L["k_proj"], h, i8).reshape(1, n, c.n_kv_heads, c.head_dim)
            v = self._linear(L["v_proj"], h, i8).reshape(1, n, c.n_kv_heads, c.head_dim)
            q, k = rope(q, start_pos, c.rope_theta), rope(k, start_pos, c.rope_theta)
            copy_to_kv_cache(k, v, self.k_cache[li], self.v_cache[li], start_pos)
            a = attention(q, self.k_cache[li], self.v_cache[li], start_pos + n).reshape(n, -1)
            res = add(res, self._linear(L["o_proj"], a, i8))
            h, _ = rmsnorm(res, L["ffn_norm"], c.rms_norm_eps)
            act = silu_mul(self._linear(L["gate_proj"], h, i8), self._linear(L["up_proj"], h, i8))
            res = add(res, self._linear(L["down_proj"], act, i8))
        h, _ = rmsnorm(res[-1:], m.final_norm, c.rms_norm_eps)
        if c.lm_head_ternary:
            return self._linear(m.lm_head, h, True)[0]
        return fp16_gemv(m.lm_head, h[0])
