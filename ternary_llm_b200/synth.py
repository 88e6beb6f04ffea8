"""Seeded synthetic ternary weights generated on the device with torch ops.

Same algorithm as pack.py (the reference's ternarize/pack.py:41-101,120-169),
written with torch so that whole models' worth of matrices can be drawn directly
in GPU memory for benchmarks.  This is input synthesis, not part of the
contraction path; tests check it against pack.py on CPU tensors.
"""
from __future__ import annotations

import torch

GROUP_SIZE = 128


def ternarize_pack(w: torch.Tensor, threshold_factor: float = 0.7):
    """float32 [N,K] (K % 128 == 0) -> (nz int32 [N,K/32], sign int32 [N,K/32],
    scales float16 [N,K/128]); int32 holds the uint32 bit patterns."""
    n, k = w.shape
    g = w.reshape(n, k // GROUP_SIZE, GROUP_SIZE)
    a = g.abs()
    thr = threshold_factor * a.mean(dim=2, keepdim=True)
    pos = g > thr
    nzm = pos | (g < -thr)
    cnt = nzm.sum(dim=2).clamp(min=1).to(torch.float32)
    scales = ((a * nzm).sum(dim=2) / cnt).to(torch.float16)
    shifts = torch.arange(32, device=w.device, dtype=torch.int64)
    nzw = (nzm.reshape(n, k // 32, 32).to(torch.int64) << shifts).sum(dim=2)
    sgw = (pos.reshape(n, k // 32, 32).to(torch.int64) << shifts).sum(dim=2)
    # wrap the 32-bit patterns into int32 storage
    nzw = torch.where(nzw >= 2 ** 31, nzw - 2 ** 32, nzw).to(torch.int32)
    sgw = torch.where(sgw >= 2 ** 31, sgw - 2 ** 32, sgw).to(torch.int32)
    return nzw.contiguous(), sgw.contiguous(), scales.contiguous()


def random_ternary_weight(rows: int, cols: int, seed: int, device, std: float = 0.02,
                          chunk_rows: int = 4096):
    """W = std * randn(rows, cols) from `seed`, ternarised and packed on `device`."""
    gen = torch.Generator(device=device).manual_seed(seed)
    nz = torch.empty(rows, cols // 32, dtype=torch.int32, device=device)
    sg = torch.empty(rows, cols // 32, dtype=torch.int32, device=device)
    sc = torch.empty(rows, cols // GROUP_SIZE, dtype=torch.float16, device=device)
    for r0 in range(0, rows, chunk_rows):
        r1 = min(rows, r0 + chunk_rows)
        w = torch.randn(r1 - r0, cols, generator=gen, device=device, dtype=torch.float32) * std
        nz[r0:r1], sg[r0:r1], sc[r0:r1] = ternarize_pack(w)
    return nz, sg, sc


def random_device_model(cfg, seed: int, device, std: float = 0.02):
    """tllm_format.random_model drawn on the device: the same structure (a TllmFile whose
    arrays are CUDA tensors), for models too large to ternarise on the host in reasonable time.
    Not bit-identical to random_model (different generator)."""
    from .tllm_format import TernaryTensor, TllmFile, pad32
    gen = torch.Generator(device=device).manual_seed(seed)

    def dense(rows, cols):
        out = torch.empty(rows, cols, dtype=torch.float16, device=device)
        for r0 in range(0, rows, 8192):
            r1 = min(rows, r0 + 8192)
            out[r0:r1] = (torch.randn(r1 - r0, cols, generator=gen, device=device) * std).to(torch.float16)
        return out

    m = TllmFile(cfg, dense(cfg.vocab_size, cfg.hidden_dim))
    for li in range(cfg.n_layers):
        layer = {}
        for pi, (name, o, i) in enumerate(cfg.proj_shapes()):
            layer[name] = TernaryTensor(*random_ternary_weight(o, i, seed=seed * 100003 + li * 16 + pi, device=device, std=std))
        layer["attn_norm"] = torch.ones(cfg.hidden_dim, dtype=torch.float16, device=device)
        layer["ffn_norm"] = torch.ones(cfg.hidden_dim, dtype=torch.float16, device=device)
        m.layers.append(layer)
    m.final_norm = torch.ones(cfg.hidden_dim, dtype=torch.float16, device=device)
    if cfg.lm_head_ternary:
        m.lm_head = TernaryTensor(*random_ternary_weight(cfg.vocab_size, pad32(cfg.hidden_dim), seed=seed * 100003 + 99991,
                                                         device=device, std=std))
    else:
        m.lm_head = dense(cfg.vocab_size, cfg.hidden_dim)
    return m
