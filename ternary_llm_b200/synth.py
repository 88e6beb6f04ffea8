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
