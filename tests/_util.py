"""Helpers shared by the GPU parity tests: exact (float64) results and the
per-element bound from the oracle, computed in row chunks to bound memory."""
import numpy as np

from oracle import oracle

REL_TOL = 2e-3   # |err| <= REL_TOL * sum_k |scale * t * x| per output element


def exact_and_bound(nz, sg, sc, x, chunk_elems=1 << 24):
    """x [B,K] or [K] float16 (or int8 times a scale given as float64 array).
    Returns (y64, bound) with the leading shape of x."""
    x = np.asarray(x)
    single = x.ndim == 1
    x2 = np.atleast_2d(x)
    n, words = nz.shape
    k = words * 32
    step = max(1, chunk_elems // k)
    ys, bs = [], []
    for r0 in range(0, n, step):
        r1 = min(n, r0 + step)
        ys.append(oracle.ternary_matvec(nz[r0:r1], sg[r0:r1], sc[r0:r1], x2, 128, np.float64))
        bs.append(oracle.tolerance_bound(nz[r0:r1], sg[r0:r1], sc[r0:r1], x2, 128, REL_TOL))
    y = np.concatenate(ys, axis=1)
    b = np.concatenate(bs, axis=1)
    return (y[0], b[0]) if single else (y, b)


def assert_within(y_gpu, y64, bound, what="", slack=0.0):
    """Checks |y_gpu - y64| <= bound (+ half an ulp of the FP16 result, which the
    bound as stated does not cover when the exact value is large and the terms
    cancel little)."""
    y_gpu = np.asarray(y_gpu, dtype=np.float64)
    err = np.abs(y_gpu - y64)
    lim = bound + slack
    bad = err > lim
    ratio = float(np.max(err / np.maximum(lim, 1e-30))) if err.size else 0.0
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} outside tolerance, worst err/tol {ratio:.3f}"
    return ratio
