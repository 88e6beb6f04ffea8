"""CPU oracle for the ternary weight-contraction path (TEST INFRASTRUCTURE ONLY).

This module restates, in numpy, the algorithms of the reference project
(jastaq/ternary-llm) that define correct results for the hot path.  It is the
checker, never the product: only tests/, __graft_entry__.smoke() and bench.py's
CPU-baseline legs may import it.  The shipped library has no CPU fallback.

Pinning: every function here is checked in tests/test_oracle.py against
  * the known-answer words of the reference's packing tests
    (tests/test_packing.py:48-89: nz 0x80000003, sign 0x80000001),
  * fixtures under tests/golden/ produced by importing the reference's own
    ternarize/pack.py and by calling the reference's compiled cpu_reference
    (tests/test_ternary_gemv.cu:40-75) -- see tests/golden/make_golden.py.
"""
from __future__ import annotations

import numpy as np

GROUP_SIZE = 128


# --------------------------------------------------------------------------
# Packing side (ternarize/pack.py)
# --------------------------------------------------------------------------
def pad_to_multiple(w: np.ndarray, multiple: int = 32) -> np.ndarray:
    """Zero-pad the last dimension up to a multiple (ternarize/pack.py:24-34)."""
    last = w.shape[-1]
    rem = last % multiple
    if rem == 0:
        return w
    pad = [(0, 0)] * (w.ndim - 1) + [(0, multiple - rem)]
    return np.pad(w, pad, mode="constant", constant_values=0)


def ternarize_tensor(weight: np.ndarray, group_size: int = GROUP_SIZE,
                     threshold_factor: float = 0.7):
    """Ternarise a float32 tensor per flat group (ternarize/pack.py:41-101).

    threshold = factor * mean|w| per group, strict comparisons (:80-86);
    scale = mean|w| over the group's nonzeros, as float16, 0 for an empty
    group (:88-93).  Returns (int8 ternary of weight's shape, float16 [numel/gs]).

    The group mean is taken in float32 like the reference's torch ops; the sum
    order inside a 128-element mean can differ from torch's by an ulp, which can
    only move a weight that sits exactly on the threshold.  Golden fixtures made
    with the reference itself pin the cases the tests use.
    """
    w = np.asarray(weight, dtype=np.float32)
    shape = w.shape
    flat = w.reshape(-1)
    numel = flat.size
    pad = (-numel) % group_size
    if pad:
        flat = np.concatenate([flat, np.zeros(pad, np.float32)])
    groups = flat.reshape(-1, group_size)
    absg = np.abs(groups)
    mean_abs = absg.mean(axis=1, keepdims=True, dtype=np.float32)
    thr = np.float32(threshold_factor) * mean_abs
    tern = np.zeros(groups.shape, np.int8)
    tern[groups > thr] = 1
    tern[groups < -thr] = -1
    nzm = tern != 0
    cnt = np.maximum(nzm.sum(axis=1), 1).astype(np.float32)
    nzsum = (absg * nzm.astype(np.float32)).sum(axis=1, dtype=np.float32)
    scales = (nzsum / cnt).astype(np.float16)
    tern = tern.reshape(-1)[:numel].reshape(shape)
    return tern, scales


def pack_ternary_to_bitmasks(ternary: np.ndarray):
    """int8 [N,K] -> (nonzero uint32 [N,K/32], sign uint32 [N,K/32]).

    Bit k of word c of row r is element [r, 32c+k]; nonzero bit = value != 0,
    sign bit = value > 0 (ternarize/pack.py:120-169).
    """
    t = np.asarray(ternary)
    assert t.ndim == 2 and t.shape[1] % 32 == 0
    n, k = t.shape
    t3 = t.reshape(n, k // 32, 32)
    shifts = (np.uint64(1) << np.arange(32, dtype=np.uint64))
    nz = ((t3 != 0).astype(np.uint64) * shifts).sum(axis=2).astype(np.uint32)
    sg = ((t3 > 0).astype(np.uint64) * shifts).sum(axis=2).astype(np.uint32)
    return nz, sg


def unpack_bitmasks(nz: np.ndarray, sg: np.ndarray) -> np.ndarray:
    """Dual bitmasks -> int8 {-1,0,+1} [N, 32*words] (tests/test_packing.py:25-41).

    A sign bit whose nonzero bit is clear decodes to 0, as in the kernels'
    pos = nz & sg, neg = nz & ~sg (kernels/ternary_gemv.cu:65-66).
    """
    nz = np.asarray(nz, dtype=np.uint32)
    sg = np.asarray(sg, dtype=np.uint32)
    n, words = nz.shape
    bits = np.arange(32, dtype=np.uint32)
    nzb = ((nz[:, :, None] >> bits) & 1).astype(np.int8)
    sgb = ((sg[:, :, None] >> bits) & 1).astype(np.int8)
    t = nzb * (2 * sgb - 1)
    return t.reshape(n, words * 32)


def unpack_bitmasks_loop(nz: np.ndarray, sg: np.ndarray) -> np.ndarray:
    """The same decode written as the reference's triple loop, for small cases
    only; used to check the vectorised form (tests/test_packing.py:25-41)."""
    n, words = nz.shape
    out = np.zeros((n, words * 32), np.int8)
    for r in range(n):
        for c in range(words):
            a, b = int(nz[r, c]), int(sg[r, c])
            for k in range(32):
                if a >> k & 1:
                    out[r, 32 * c + k] = 1 if (b >> k & 1) else -1
    return out


# --------------------------------------------------------------------------
# Contraction side
# --------------------------------------------------------------------------
def dequantize(nz, sg, scales_f16, group_size: int = GROUP_SIZE) -> np.ndarray:
    """W[n,k] = float32(scale[n, k//gs]) * t[n,k]  (include/model.h:12-21)."""
    t = unpack_bitmasks(nz, sg).astype(np.float32)
    n, k = t.shape
    s = np.asarray(scales_f16).reshape(n, k // group_size).astype(np.float32)
    return t * np.repeat(s, group_size, axis=1)


def ternary_matvec(nz, sg, scales_f16, x_f16, group_size: int = GROUP_SIZE,
                   dtype=np.float32) -> np.ndarray:
    """y[b,n] = sum_g scale[n,g] * sum_{k in g} t[n,k] * x[b,k].

    Follows cpu_reference (tests/test_ternary_gemv.cu:40-75): group sums first,
    then the scale, accumulated in `dtype` (float32 like the reference; pass
    float64 for the exact value used in the tolerance check).  x may be [K]
    or [B,K]; the result has the matching leading shape.
    """
    x = np.asarray(x_f16)
    single = x.ndim == 1
    x2 = np.atleast_2d(x).astype(dtype)
    t = unpack_bitmasks(nz, sg)
    n, k = t.shape
    g = k // group_size
    s = np.asarray(scales_f16).reshape(n, g).astype(dtype)
    out = np.zeros((x2.shape[0], n), dtype)
    t3 = t.reshape(n, g, group_size).astype(dtype)
    for b in range(x2.shape[0]):
        xg = x2[b].reshape(g, group_size)
        gs = np.einsum("ngk,gk->ng", t3, xg)
        out[b] = (gs * s).sum(axis=1, dtype=dtype)
    return out[0] if single else out


def tolerance_bound(nz, sg, scales_f16, x_f16, group_size: int = GROUP_SIZE,
                    rel: float = 2e-3) -> np.ndarray:
    """Per-output bound rel * sum_k |scale[n,k//gs] * t[n,k] * x[k]| in float64.

    This is the nonzero-only (tighter) reading of "|err| <= 2e-3 * sum|scale*x|".
    """
    x = np.asarray(x_f16)
    single = x.ndim == 1
    x2 = np.abs(np.atleast_2d(x).astype(np.float64))
    t = np.abs(unpack_bitmasks(nz, sg)).astype(np.float64)
    n, k = t.shape
    g = k // group_size
    s = np.abs(np.asarray(scales_f16).reshape(n, g).astype(np.float64))
    w = t * np.repeat(s, group_size, axis=1)
    out = rel * (x2 @ w.T)
    return out[0] if single else out


def ternary_gemm(a_f16, nz, sg, scales_f16, group_size: int = GROUP_SIZE,
                 dtype=np.float32) -> np.ndarray:
    """C[M,N] = A[M,K] . W^T with W dequantised (kernels/ternary_gemm.cu:4-11)."""
    return ternary_matvec(nz, sg, scales_f16, np.asarray(a_f16), group_size, dtype)


def quantize_absmax_int8(x_f16):
    """half[n] -> (int8[n], float scale)  (kernels/activations.cu:88-142).

    absmax in float32; scale = absmax/127, or 1.0 when absmax == 0;
    q = clamp(rint(x * (127/absmax)), -127, 127) with round-half-even
    (__float2int_rn, :138); an all-zero input gives zeros.
    """
    x = np.asarray(x_f16).astype(np.float32)
    absmax = np.float32(np.max(np.abs(x))) if x.size else np.float32(0)
    if absmax > 0:
        scale = np.float32(absmax / np.float32(127.0))
        inv = np.float32(np.float32(127.0) / absmax)
    else:
        scale = np.float32(1.0)
        inv = np.float32(0.0)
    q = np.rint(x * inv)
    q = np.clip(q, -127, 127).astype(np.int8)
    return q, scale


def ternary_matvec_int8(nz, sg, scales_f16, x_i8, input_scale: float,
                        group_size: int = GROUP_SIZE, dtype=np.float32) -> np.ndarray:
    """y[n] = input_scale * sum_g scale[n,g] * (exact integer group sum)
    (kernels/ternary_gemv.cu:116-199)."""
    t = unpack_bitmasks(nz, sg).astype(np.int32)
    n, k = t.shape
    g = k // group_size
    xi = np.asarray(x_i8).astype(np.int32).reshape(g, group_size)
    gsum = np.einsum("ngk,gk->ng", t.reshape(n, g, group_size), xi)
    s = np.asarray(scales_f16).reshape(n, g).astype(dtype)
    acc = (s * gsum.astype(dtype)).sum(axis=1, dtype=dtype)
    return (acc * dtype(input_scale)).astype(dtype)


def tolerance_bound_int8(nz, sg, scales_f16, x_i8, input_scale: float,
                         group_size: int = GROUP_SIZE, rel: float = 2e-3) -> np.ndarray:
    """Same bound as tolerance_bound with x = input_scale * x_int8."""
    xf = np.asarray(x_i8).astype(np.float64) * float(input_scale)
    return tolerance_bound(nz, sg, scales_f16, xf, group_size, rel)


# --------------------------------------------------------------------------
# Synthetic inputs with the distribution the benchmark configurations state
# --------------------------------------------------------------------------
def make_case(n: int, k: int, seed: int, batch: int = 1, random_masks: bool = False,
              signed_scales: bool = False):
    """Seeded inputs: W = 0.02*randn(N,K) ternarised per 128 along K (about 42 %
    zeros), x = randn(B,K) as float16.  random_masks=True draws independent
    random words for both masks, with scales U(-0.1,0.1) when signed_scales, as
    the reference's GPU test does (tests/test_ternary_gemv.cu:98-108)."""
    rng = np.random.default_rng(seed)
    if random_masks:
        nz = rng.integers(0, 2**32, size=(n, k // 32), dtype=np.uint64).astype(np.uint32)
        sg = rng.integers(0, 2**32, size=(n, k // 32), dtype=np.uint64).astype(np.uint32)
        lo = -0.1 if signed_scales else 0.0
        sc = rng.uniform(lo, 0.1, size=(n, k // GROUP_SIZE)).astype(np.float16)
    else:
        w = (0.02 * rng.standard_normal((n, k))).astype(np.float32)
        t, sc = ternarize_tensor(w, GROUP_SIZE, 0.7)
        nz, sg = pack_ternary_to_bitmasks(t)
        sc = sc.reshape(n, k // GROUP_SIZE)
    x = rng.standard_normal((batch, k)).astype(np.float16)
    return nz, sg, sc, x
