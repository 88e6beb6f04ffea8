"""GPU parity at the sizes the benchmark definition names: the LLaMA-3-8B projection shapes
at batch 4 and 16, the prefill GEMM at the gate/up and down shapes for 128 / 512 / 2048
tokens, and the per-rank shapes of the LLaMA-70B tensor-parallel split on one GPU.

Weights are drawn on the device (seeded); the oracle (float64, the 2e-3 * sum|scale*t*x|
bound plus half an FP16 ulp) is evaluated on a sample of output rows that always holds the
first and the last 64 rows and the rows either side of every 1/37 of the matrix, which
is where a row block changes hands between CTAs.  Every output, sampled or not, must be
finite and -- a size-independent property -- doubling the activations must double every
output exactly.
"""
import numpy as np
import pytest
import torch

import ternary_llm_b200 as tl
from ternary_llm_b200 import synth
from tests._util import assert_within, exact_and_bound

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

SHAPES_8B = {"q/o": (4096, 4096), "k/v": (1024, 4096), "gate/up": (14336, 4096), "down": (4096, 14336)}


def _half_ulp(y64):
    a = np.maximum(np.abs(y64), 2.0 ** -14)
    return 0.5 * 2.0 ** (np.floor(np.log2(a)) - 10)


def _sample_rows(n, count=384, seed=0):
    rows = set(range(min(64, n))) | set(range(max(0, n - 64), n))
    for i in range(1, 37):                      # neighbourhoods of evenly spread cut points
        c = n * i // 37
        rows |= {r for r in (c - 1, c, c + 1) if 0 <= r < n}
    rng = np.random.default_rng(seed)
    rows |= set(int(r) for r in rng.integers(0, n, count))
    return np.array(sorted(rows))


def _weights(n, k, seed):
    torch.cuda.set_device(0)
    nz, sg, sc = synth.random_ternary_weight(n, k, seed=seed, device=torch.device(DEV))
    w = tl.PreparedWeight(nz, sg, sc, n, k, register=False)
    return nz, sg, sc, w


def _host_rows(nz, sg, sc, rows):
    idx = torch.from_numpy(rows).to(DEV)
    return (nz[idx].cpu().numpy().view(np.uint32), sg[idx].cpu().numpy().view(np.uint32), sc[idx].cpu().numpy())


def _check_rows(y_gpu, nz, sg, sc, rows, x, what):
    """y_gpu [B, N] float16 numpy; x [B, K] float16 numpy."""
    hnz, hsg, hsc = _host_rows(nz, sg, sc, rows)
    y64, bound = exact_and_bound(hnz, hsg, hsc, x)
    assert np.isfinite(y_gpu).all(), f"{what}: non-finite outputs"
    return assert_within(y_gpu[:, rows], y64, bound, what, slack=_half_ulp(y64))


@pytest.mark.parametrize("batch", [4, 16])
@pytest.mark.parametrize("name", list(SHAPES_8B))
def test_gemv_batched_at_8b_shapes(name, batch):
    n, k = SHAPES_8B[name]
    nz, sg, sc, w = _weights(n, k, seed=1000 + n + k)
    x = np.random.default_rng(batch + n).standard_normal((batch, k)).astype(np.float16)
    dx = torch.from_numpy(x).to(DEV)
    y = torch.full((batch, n), float("nan"), dtype=torch.float16, device=DEV)
    tl.ternary_gemv_packed(w, dx, y, batch)
    y2 = torch.full((batch, n), float("nan"), dtype=torch.float16, device=DEV)
    tl.ternary_gemv_packed(w, (dx.float() * 2).half(), y2, batch)
    torch.cuda.synchronize()
    tl.check_device_errors()
    _check_rows(y.cpu().numpy(), nz, sg, sc, _sample_rows(n, seed=batch), x, f"gemv {name} batch {batch}")
    if batch <= 8:      # the integer-MMA GEMV: scaling by two only shifts the block exponent
        # (exact wherever the FP16 result is a normal number; a subnormal one rounds on a fixed grid)
        normal = y.float().abs() >= 2.0 ** -13
        assert torch.equal(y2.float()[normal], y.float()[normal] * 2), "W(2x) != 2 W(x)"
        assert bool(((y2.float() - 2 * y.float()).abs() <= 2.0 ** -23).all())
    else:               # the tcgen05 route: FP16 x FP16 products summed in hardware, to one last place
        d = (y2.float() - 2 * y.float()).abs()
        assert bool((d <= (2 * y.float()).abs() * 2.0 ** -10 + 1e-6).all()), "W(2x) differs from 2 W(x) by more than one ulp"


GEMM_CASES = [(m, s) for s in ("gate/up", "down") for m in (128, 512, 2048)] + [(2048, "k/v"), (2048, "q/o")]


@pytest.mark.parametrize("m,name", GEMM_CASES)
def test_gemm_at_8b_shapes(m, name):
    """The tcgen05 GEMM at the prefill sizes of the benchmark definition (k/v at 2048 tokens
    takes the split-K path), sampled tokens x sampled features against the oracle."""
    n, k = SHAPES_8B[name]
    nz, sg, sc, w = _weights(n, k, seed=2000 + n + k)
    a = torch.randn(m, k, device=DEV, generator=torch.Generator(device=DEV).manual_seed(m)).half()
    c = torch.full((m, n), float("nan"), dtype=torch.float16, device=DEV)
    tl.ternary_gemm_packed(a, w, c, m)
    torch.cuda.synchronize()
    tl.check_device_errors()
    assert bool(torch.isfinite(c).all())
    toks = np.unique(np.concatenate([[0, m - 1, m // 2, 255 % m, 256 % m],
                                     np.random.default_rng(m).integers(0, m, 6)]))
    rows = _sample_rows(n, count=256, seed=m)
    x = a[torch.from_numpy(toks).to(DEV)].cpu().numpy()
    cg = c[torch.from_numpy(toks).to(DEV)].cpu().numpy()
    _check_rows(cg, nz, sg, sc, rows, x, f"gemm M={m} {name}")


def _tp_shapes():
    out = [(8192, 8192), (8192, 28672), (28672, 8192)]
    for tp in (2, 4, 8):
        out += [(28672 // tp, 8192), (8192, 28672 // tp), (8192, 8192 // tp), (8192 // tp, 8192), (1024 // tp, 8192)]
    return sorted(set(out))


@pytest.mark.parametrize("n,k", _tp_shapes())
def test_gemv_at_70b_shard_shapes(n, k):
    """Every matrix shape one rank of the LLaMA-70B tensor-parallel split streams (tp = 2, 4,
    8), and the unsharded shapes, batch 1, FP16 and INT8 activations."""
    nz, sg, sc, w = _weights(n, k, seed=3000 + n + k)
    x = np.random.default_rng(n + k).standard_normal((1, k)).astype(np.float16)
    dx = torch.from_numpy(x).to(DEV)
    y = torch.full((1, n), float("nan"), dtype=torch.float16, device=DEV)
    tl.ternary_gemv_packed(w, dx, y, 1)
    q = torch.zeros(k, dtype=torch.int8, device=DEV)
    scale = torch.zeros(1, dtype=torch.float32, device=DEV)
    tl.quantize_absmax_int8(dx[0], q, scale, k)
    yi = torch.full((n,), float("nan"), dtype=torch.float16, device=DEV)
    tl.ternary_gemv_int8_packed(w, q, float(scale.item()), yi)
    torch.cuda.synchronize()
    tl.check_device_errors()
    rows = _sample_rows(n, seed=k)
    _check_rows(y.cpu().numpy(), nz, sg, sc, rows, x, f"gemv {n}x{k}")
    xq = (q.cpu().numpy().astype(np.float64) * float(scale.item()))[None, :]
    hnz, hsg, hsc = _host_rows(nz, sg, sc, rows)
    y64, bound = exact_and_bound(hnz, hsg, hsc, xq)
    got = yi.cpu().numpy()
    assert np.isfinite(got).all()
    assert_within(got[None, rows], y64, bound, f"gemv int8 {n}x{k}", slack=_half_ulp(y64))


def test_gemv_config0_shape():
    """The single-GEMV configuration: K = 2048, N = 8192 (the 1B up-projection)."""
    n, k = 8192, 2048
    nz, sg, sc, w = _weights(n, k, seed=7)
    x = np.random.default_rng(7).standard_normal((1, k)).astype(np.float16)
    y = torch.full((1, n), float("nan"), dtype=torch.float16, device=DEV)
    tl.ternary_gemv_packed(w, torch.from_numpy(x).to(DEV), y, 1)
    torch.cuda.synchronize()
    _check_rows(y.cpu().numpy(), nz, sg, sc, np.arange(n), x, "config 0")


def test_non_finite_activations_reach_the_output():
    """FP32 accumulation of x, as the reference does it, carries a NaN or an infinity into
    the result; the block-fixed-point staging must not hide one.  Here a scale group that
    holds a non-finite activation makes every output NaN (the dequantise-then-multiply
    oracle gives NaN or an infinity in those outputs); a vector without one is untouched."""
    n, k = 192, 512
    nz, sg, sc, w = _weights(n, k, seed=9)
    x = np.random.default_rng(9).standard_normal((3, k)).astype(np.float16)
    x[0, 130] = np.nan
    x[1, 300] = np.inf
    dx = torch.from_numpy(x).to(DEV)
    for batch in (1, 2, 3):
        y = torch.zeros(batch, n, dtype=torch.float16, device=DEV)
        tl.ternary_gemv_packed(w, dx[:batch].contiguous(), y, batch)
        torch.cuda.synchronize()
        assert bool(torch.isnan(y[0]).all())
        if batch > 1:
            assert bool(torch.isnan(y[1]).all())
        if batch > 2:
            rows = np.arange(n)
            _check_rows(y.cpu().numpy()[2:3], nz, sg, sc, rows, x[2:3], "finite vector beside non-finite ones")
    # one vector alone with the non-finite value: same
    y = torch.zeros(1, n, dtype=torch.float16, device=DEV)
    tl.ternary_gemv_packed(w, dx[1:2].contiguous(), y, 1)
    torch.cuda.synchronize()
    assert bool(torch.isnan(y).all())


def test_three_and_four_vectors_per_pass_keep_the_benchmark_bound_on_outliers():
    """Batches of three and four vectors share one MMA column block on 16-bit block fixed
    point per scale group (one and two vectors ride 24 bits).  Its rounding error per output
    is at most 2^-17 * sum_g scale * 128 * max|x_g|, which stays below the benchmark's bound
    2e-3 * sum_k |scale * x_k| (every k of the row) whatever the input; the tighter reading
    used everywhere else in this suite (nonzero weights only) holds on ordinary data but can
    be exceeded where a group's one huge activation meets a zero weight.  Both are checked."""
    n, k = 256, 1024
    nz, sg, sc, w = _weights(n, k, seed=77)
    rng = np.random.default_rng(77)
    for batch in (3, 4):
        x = rng.standard_normal((batch, k)).astype(np.float32)
        x[0, 5] = 60000.0                # one huge activation in a group of ordinary ones
        x[2, 130] = -1.9995              # mantissa at the top: the group takes one exponent more
        x = x.astype(np.float16)
        y = torch.full((batch, n), float("nan"), dtype=torch.float16, device=DEV)
        tl.ternary_gemv_packed(w, torch.from_numpy(x).to(DEV), y, batch)
        torch.cuda.synchronize()
        got = y.cpu().numpy().astype(np.float64)
        rows = np.arange(n)
        hnz, hsg, hsc = _host_rows(nz, sg, sc, rows)
        y64, tight = exact_and_bound(hnz, hsg, hsc, x)
        gsum = np.abs(x.astype(np.float64)).reshape(batch, k // 128, 128).sum(axis=2)
        literal = 2e-3 * gsum @ hsc.astype(np.float64).T + _half_ulp(y64)
        err = np.abs(got - y64)
        assert (err <= literal).all(), f"batch {batch}: beyond 2e-3 * sum|scale * x| by {np.max(err / literal):.3g}"
        assert (err[1:] <= tight[1:] + _half_ulp(y64[1:])).all(), "ordinary vectors beside the outlier"


@pytest.mark.parametrize("n,k", [(3560, 14336), (2384, 28672), (4096, 12288)])
def test_column_split_launches_with_ragged_row_counts(n, k):
    """Long rows run as clusters of two CTAs that split the columns (each stages one half of
    the activations, the halves' sums meet in shared memory).  Row counts that leave a partial
    last row block and an uneven number of row blocks per cluster, against the oracle; a second
    call must give the same bits (the exchange buffers carry nothing over)."""
    nz, sg, sc, w = _weights(n, k, seed=4000 + n)
    x = np.random.default_rng(n).standard_normal((1, k)).astype(np.float16)
    dx = torch.from_numpy(x).to(DEV)
    y = torch.full((1, n), float("nan"), dtype=torch.float16, device=DEV)
    y2 = torch.full((1, n), float("nan"), dtype=torch.float16, device=DEV)
    tl.ternary_gemv_packed(w, dx, y, 1)
    tl.ternary_gemv_packed(w, dx, y2, 1)
    torch.cuda.synchronize()
    tl.check_device_errors()
    assert torch.equal(y, y2)
    _check_rows(y.cpu().numpy(), nz, sg, sc, _sample_rows(n, seed=k), x, f"column split {n}x{k}")


def test_column_split_with_matrices_packed_back_to_back():
    """Two matrices that share a long input vector, streamed as one launch (the fused gate|up
    form) through the column-split path: every row lands in its own output."""
    k, ns = 14336, (2048, 2064)
    torch.cuda.set_device(0)
    src = [synth.random_ternary_weight(n, k, seed=5000 + i, device=torch.device(DEV)) + (n, k) for i, n in enumerate(ns)]
    ws = tl.prepare_group(src, keep_source=True)
    x = np.random.default_rng(5).standard_normal((1, k)).astype(np.float16)
    dx = torch.from_numpy(x).to(DEV)
    ys = [torch.full((n,), float("nan"), dtype=torch.float16, device=DEV) for n in ns]
    tl.ternary_gemv_packed_multi(ws, dx[0], ys)
    torch.cuda.synchronize()
    tl.check_device_errors()
    for (nz, sg, sc, n, _), y in zip(src, ys):
        _check_rows(y.cpu().numpy()[None, :], nz, sg, sc, _sample_rows(n, seed=n), x, f"grouped column split, {n} rows")


@pytest.mark.parametrize("k,ns,with_residual", [(4096, (4096, 1024, 1024), True), (8192, (3584, 3584), True),
                                                (2048, (8192,), False), (4096, (512, 528), True)])
def test_gemv_with_residual_add_and_rmsnorm_staged_in_the_launch(k, ns, with_residual):
    """ternary_gemv_packed_multi_norm: x = rmsnorm(a + b) * w is made inside the GEMV launch.
    The rounded sum must come out bit for bit, and the projections must match the oracle
    applied to the oracle's own add + rmsnorm of the same inputs."""
    from oracle import layer_oracle as LO
    torch.cuda.set_device(0)
    src = [synth.random_ternary_weight(n, k, seed=6000 + i + k, device=torch.device(DEV)) + (n, k) for i, n in enumerate(ns)]
    ws = tl.prepare_group(src, keep_source=True) if len(ns) > 1 else [tl.PreparedWeight(*src[0], register=False)]
    rng = np.random.default_rng(k)
    a = rng.standard_normal(k).astype(np.float16)
    b = (3.0 * rng.standard_normal(k)).astype(np.float16) if with_residual else None
    w = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float16)
    eps = 1e-5
    s16 = (a.astype(np.float32) + b.astype(np.float32)).astype(np.float16) if with_residual else a
    h, _ = LO.rmsnorm(s16[None, :], w, eps)
    da, dw = torch.from_numpy(a).to(DEV), torch.from_numpy(w).to(DEV)
    db = torch.from_numpy(b).to(DEV) if with_residual else None
    res = torch.full((k,), float("nan"), dtype=torch.float16, device=DEV) if with_residual else None
    ys = [torch.full((n,), float("nan"), dtype=torch.float16, device=DEV) for n in ns]
    tl.ternary_gemv_packed_multi_norm(ws, da, db, dw, res, eps, ys)
    torch.cuda.synchronize()
    tl.check_device_errors()
    if with_residual:
        assert np.array_equal(res.cpu().numpy().view(np.uint16), s16.view(np.uint16)), "residual sum"
        with pytest.raises(ValueError):
            tl.ternary_gemv_packed_multi_norm(ws, da, db, dw, da, eps, ys)
    # the kernel's rsqrtf and the oracle's 1/sqrt may differ in the last FP16 place of x: compare
    # through the bound on the oracle's x plus the effect of one ulp of x
    for (nz, sg, sc, n, _), y in zip(src, ys):
        rows = _sample_rows(n, seed=n)
        hnz, hsg, hsc = _host_rows(nz, sg, sc, rows)
        y64, bound = exact_and_bound(hnz, hsg, hsc, h.astype(np.float16))
        ulp_x = np.abs(h.astype(np.float64)) * 2.0 ** -10
        extra = exact_and_bound(hnz, hsg, hsc, ulp_x.astype(np.float16))[1] / 2e-3      # sum |scale * t| * ulp(x)
        got = y.cpu().numpy().astype(np.float64)[None, rows]
        assert np.isfinite(got).all()
        assert (np.abs(got - y64) <= bound + extra + _half_ulp(y64)).all(), f"{n} rows of {ns}, K={k}"


def test_random_shapes_and_batches_against_the_oracle():
    """Forty seeded (rows, columns, vectors) draws -- odd row counts, one to eight vectors, short
    and long rows, few and many row blocks -- through tllm_b200_gemv_packed, every output of the
    small ones and sampled rows of the large ones against the oracle."""
    rng = np.random.default_rng(2026)
    draws = []
    for _ in range(30):
        draws.append((int(rng.integers(1, 700)), 128 * int(rng.integers(1, 17)), int(rng.integers(1, 9))))
    for _ in range(10):          # large: many row blocks per CTA, long rows, partial last row block
        draws.append((int(rng.integers(2400, 9000)), 128 * int(rng.choice([16, 32, 56, 64, 96, 112, 224])),
                      int(rng.choice([1, 1, 2, 3, 4]))))
    for n, k, batch in draws:
        nz, sg, sc, w = _weights(n, k, seed=n * 31 + k)
        x = rng.standard_normal((batch, k)).astype(np.float16)
        y = torch.full((batch, n), float("nan"), dtype=torch.float16, device=DEV)
        tl.ternary_gemv_packed(w, torch.from_numpy(x).to(DEV), y, batch)
        torch.cuda.synchronize()
        rows = np.arange(n) if n <= 700 else _sample_rows(n, count=128, seed=k)
        _check_rows(y.cpu().numpy(), nz, sg, sc, rows, x, f"random draw {n}x{k} batch {batch}")
    tl.check_device_errors()
