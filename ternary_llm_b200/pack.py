"""Ternarise and pack weights into the reference's dual-bitmask layout (host side).

Same function names, arguments and results as the reference's ternarize/pack.py
(pad_to_multiple :24-34, ternarize_tensor :41-101, pack_ternary_to_bitmasks
:120-169), on numpy arrays.  Used to make seeded synthetic weights for tests and
benchmarks and by the .tllm writer; the GPU kernels never call it.
"""
from __future__ import annotations

import numpy as np

GROUP_SIZE = 128


def pad_to_multiple(w: np.ndarray, multiple: int = 32) -> np.ndarray:
    rem = w.shape[-1] % multiple
    if rem == 0:
        return w
    width = [(0, 0)] * (w.ndim - 1) + [(0, multiple - rem)]
    return np.pad(w, width)


def ternarize_tensor(weight: np.ndarray, group_size: int = GROUP_SIZE, threshold_factor: float = 0.7):
    """float32 tensor -> (int8 {-1,0,+1} of the same shape, float16 scales [numel/gs]).

    Groups are taken over the flattened tensor; dead zone = factor * mean|w| of the
    group with strict comparisons; scale = mean|w| over the group's nonzeros (0 when
    the group is empty)."""
    w = np.ascontiguousarray(weight, dtype=np.float32)
    flat = w.reshape(-1)
    numel = flat.size
    pad = (-numel) % group_size
    if pad:
        flat = np.concatenate([flat, np.zeros(pad, np.float32)])
    g = flat.reshape(-1, group_size)
    a = np.abs(g)
    thr = np.float32(threshold_factor) * a.mean(axis=1, keepdims=True, dtype=np.float32)
    t = (g > thr).astype(np.int8) - (g < -thr).astype(np.int8)
    nzm = t != 0
    cnt = np.maximum(nzm.sum(axis=1), 1).astype(np.float32)
    scales = ((a * nzm).sum(axis=1, dtype=np.float32) / cnt).astype(np.float16)
    return t.reshape(-1)[:numel].reshape(w.shape), scales


def pack_ternary_to_bitmasks(ternary: np.ndarray):
    """int8 [N,K] (K % 32 == 0) -> (nonzero uint32 [N,K/32], sign uint32 [N,K/32]);
    bit k of word c of row r is element [r, 32c+k]."""
    t = np.asarray(ternary)
    if t.ndim != 2 or t.shape[1] % 32:
        raise ValueError("expected a 2-D tensor whose last dimension is a multiple of 32")
    n, k = t.shape
    nzb = np.packbits((t != 0).reshape(n, k // 32, 32), axis=2, bitorder="little")
    sgb = np.packbits((t > 0).reshape(n, k // 32, 32), axis=2, bitorder="little")
    return (np.ascontiguousarray(nzb).view("<u4").reshape(n, k // 32),
            np.ascontiguousarray(sgb).view("<u4").reshape(n, k // 32))


def unpack_bitmasks(nonzero_masks: np.ndarray, sign_masks: np.ndarray) -> np.ndarray:
    """Inverse of pack_ternary_to_bitmasks; a sign bit without its nonzero bit is 0."""
    nz = np.ascontiguousarray(nonzero_masks, dtype="<u4")
    sg = np.ascontiguousarray(sign_masks, dtype="<u4")
    n, words = nz.shape
    a = np.unpackbits(nz.view(np.uint8).reshape(n, words * 4), axis=1, bitorder="little").astype(np.int8)
    s = np.unpackbits(sg.view(np.uint8).reshape(n, words * 4), axis=1, bitorder="little").astype(np.int8)
    return a * (2 * s - 1)


def random_ternary_weight(rows: int, cols: int, seed: int, std: float = 0.02):
    """Seeded synthetic matrix with the benchmark's distribution: W = std*randn,
    ternarised per 128 along K (about 42 % zeros).  Returns (nz, sign, scales[rows, cols/128])."""
    rng = np.random.default_rng(seed)
    nz = np.empty((rows, cols // 32), np.uint32)
    sg = np.empty((rows, cols // 32), np.uint32)
    sc = np.empty((rows, cols // GROUP_SIZE), np.float16)
    step = max(1, (1 << 22) // cols)
    for r0 in range(0, rows, step):
        r1 = min(rows, r0 + step)
        w = rng.standard_normal((r1 - r0, cols), dtype=np.float32) * np.float32(std)
        t, s = ternarize_tensor(w, GROUP_SIZE, 0.7)
        nz[r0:r1], sg[r0:r1] = pack_ternary_to_bitmasks(t)
        sc[r0:r1] = s.reshape(r1 - r0, cols // GROUP_SIZE)
    return nz, sg, sc
