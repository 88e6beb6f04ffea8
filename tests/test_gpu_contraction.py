"""GPU parity tests: every entry point of the C ABI against the CPU oracle.

Tolerance (stated by the benchmark definition): |y - y_exact| <= 2e-3 * sum_k
|scale*t*x| per output element, y_exact computed in float64 by the oracle; plus
half an FP16 ulp of the result for the final rounding.  Integer outputs (the
INT8 quantiser) are compared bit for bit.
"""
import os

import numpy as np
import pytest
import torch

import ternary_llm_b200 as tl
from oracle import cpu, oracle
from tests._util import assert_within, exact_and_bound

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _dev(a):
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).to(DEV)
    return torch.from_numpy(a).to(DEV)


def _half_ulp(y64):
    a = np.maximum(np.abs(y64), 2.0 ** -14)
    return 0.5 * 2.0 ** (np.floor(np.log2(a)) - 10)


def _run_gemv(nz, sg, sc, x):
    n, k = nz.shape[0], nz.shape[1] * 32
    b = x.shape[0]
    dnz, dsg, dsc, dx = _dev(nz), _dev(sg), _dev(sc), _dev(x)
    y = torch.full((b, n), float("nan"), dtype=torch.float16, device=DEV)
    if b == 1:
        tl.ternary_gemv(dnz, dsg, dsc, dx, y, n, k)
    else:
        tl.ternary_gemv_batched(dnz, dsg, dsc, dx, y, b, n, k)
    torch.cuda.synchronize()
    return y.cpu().numpy()


@pytest.mark.parametrize("n,k", [(1, 128), (9, 128), (16, 256), (33, 384), (64, 1024), (1024, 1024),
                                 (1000, 2048), (4096, 4096), (4096, 11008), (8192, 2048)])
def test_gemv_fp16_vs_oracle(n, k):
    nz, sg, sc, x = oracle.make_case(n, k, seed=n * 7 + k)
    y = _run_gemv(nz, sg, sc, x)
    y64, bound = exact_and_bound(nz, sg, sc, x)
    assert not np.isnan(y).any()
    assert_within(y, y64, bound, f"gemv {n}x{k}", slack=_half_ulp(y64))


@pytest.mark.parametrize("n,k", [(16, 128), (48, 512), (1024, 1024), (4096, 4096)])
def test_gemv_random_words_signed_scales(n, k):
    # independent random mask words (sign bits without nonzero bits) and scales of
    # both signs, as the reference's GPU test draws them (tests/test_ternary_gemv.cu:98-108)
    nz, sg, sc, x = oracle.make_case(n, k, seed=11 + n, random_masks=True, signed_scales=True)
    y = _run_gemv(nz, sg, sc, x)
    y64, bound = exact_and_bound(nz, sg, sc, x)
    assert_within(y, y64, bound, f"gemv random {n}x{k}", slack=_half_ulp(y64))
    # the reference's own acceptance test (tests/test_ternary_gemv.cu:160-161)
    yref = cpu.matvec_f16(nz, sg, sc, x[0])
    err = np.abs(y[0].astype(np.float32) - yref)
    assert err.max() < 1e-2 or (err / np.maximum(np.abs(yref), 1e-6)).max() < 1e-2


def test_gemv_golden_fixtures(golden_dir):
    z = np.load(os.path.join(golden_dir, "matvec.npz"))
    for case in sorted({k.split("/")[0] for k in z.files}):
        nz, sg, sc, x, yref = (z[f"{case}/{f}"] for f in ("nz", "sign", "scales", "x", "y"))
        y = _run_gemv(nz, sg, sc, x[None, :])[0]
        y64, bound = exact_and_bound(nz, sg, sc, x)
        assert_within(y, y64, bound, case, slack=_half_ulp(y64))
        # and against the reference's own float32 result, to FP16 rounding of it
        assert np.abs(y.astype(np.float64) - yref).max() <= (bound + _half_ulp(y64)).max()


@pytest.mark.parametrize("batch", [1, 2, 3, 4, 5, 8, 13, 16])
def test_gemv_batched(batch):
    n, k = 528, 1024
    nz, sg, sc, x = oracle.make_case(n, k, seed=100 + batch, batch=batch)
    y = _run_gemv(nz, sg, sc, x)
    y64, bound = exact_and_bound(nz, sg, sc, x)
    assert_within(y, y64, bound, f"batched B={batch}", slack=_half_ulp(y64))


def test_gemv_edge_values():
    n, k = 32, 512
    nz, sg, sc, x = oracle.make_case(n, k, seed=5)
    nz[3] = 0                      # an all-zero row
    sc[4] = 0                      # zero scales
    sc[5] = -sc[5]                 # negative scales
    nz[6], sg[6] = 0xFFFFFFFF, 0xFFFFFFFF   # all +1
    nz[7], sg[7] = 0xFFFFFFFF, 0            # all -1
    sg[8] = 0xFFFFFFFF             # sign bits everywhere, nonzero bits unchanged
    y = _run_gemv(nz, sg, sc, x)
    y64, bound = exact_and_bound(nz, sg, sc, x)
    assert y[0, 3] == 0 and y[0, 4] == 0
    assert_within(y, y64, bound, "edge", slack=_half_ulp(y64))


@pytest.mark.parametrize("n", [1, 7, 255, 256, 4096, 14336, 28672, 40000])
def test_quantize_absmax_int8_bit_exact(n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n).astype(np.float16)
    dx = _dev(x)
    q = torch.zeros(n, dtype=torch.int8, device=DEV)
    s = torch.zeros(1, dtype=torch.float32, device=DEV)
    tl.quantize_absmax_int8(dx, q, s, n)
    torch.cuda.synchronize()
    qo, so = oracle.quantize_absmax_int8(x)
    assert s.item() == float(so)
    assert (q.cpu().numpy() == qo).all()


def test_quantize_zero_and_ties():
    x = np.zeros(256, np.float16)
    q = torch.ones(256, dtype=torch.int8, device=DEV)
    s = torch.zeros(1, dtype=torch.float32, device=DEV)
    tl.quantize_absmax_int8(_dev(x), q, s, 256)
    assert s.item() == 1.0 and (q.cpu().numpy() == 0).all()
    # absmax 127 -> factor exactly 1: halves k + 0.5 are ties and round to even
    x = np.array([127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 63.5], np.float16)
    q = torch.zeros(8, dtype=torch.int8, device=DEV)
    tl.quantize_absmax_int8(_dev(x), q, s, 8)
    assert q.cpu().numpy().tolist() == [127, 0, 2, 2, 0, -2, -2, 64]
    assert s.item() == 1.0


@pytest.mark.parametrize("n,k", [(16, 128), (100, 512), (1024, 1024), (4096, 4096), (4096, 11008)])
def test_gemv_int8_vs_oracle(n, k):
    nz, sg, sc, x = oracle.make_case(n, k, seed=n + k, random_masks=(n == 100), signed_scales=True)
    q, s = oracle.quantize_absmax_int8(x[0])
    y = torch.zeros(n, dtype=torch.float16, device=DEV)
    tl.ternary_gemv_int8(_dev(nz), _dev(sg), _dev(sc), _dev(q), float(s), y, n, k)
    torch.cuda.synchronize()
    xs = q.astype(np.float64) * np.float64(s)
    y64 = oracle.ternary_matvec(nz, sg, sc, xs, 128, np.float64)
    bound = oracle.tolerance_bound(nz, sg, sc, xs, 128)
    assert_within(y.cpu().numpy(), y64, bound, f"int8 {n}x{k}", slack=_half_ulp(y64))


@pytest.mark.parametrize("n,k", [(1024, 1024), (4096, 4096), (4096, 11008)])
def test_reference_acceptance_tests(n, k):
    """The reference's own GPU test, restated: its shapes, input distributions
    (uniform words, scales U(-0.1,0.1), activations U(-1,1)) and pass criteria
    (tests/test_ternary_gemv.cu:98-116,160-161,270-271)."""
    rng = np.random.default_rng(n + k)
    nz = rng.integers(0, 2**32, size=(n, k // 32), dtype=np.uint64).astype(np.uint32)
    sg = rng.integers(0, 2**32, size=(n, k // 32), dtype=np.uint64).astype(np.uint32)
    sc_f = rng.uniform(-0.1, 0.1, size=(n, k // 128)).astype(np.float32)
    x_f = rng.uniform(-1, 1, size=k).astype(np.float32)
    sc, x = sc_f.astype(np.float16), x_f.astype(np.float16)
    yref = cpu.matvec_f32(nz, sg, sc_f, x_f, 128, threads=0)        # un-rounded inputs, as the reference does
    dnz, dsg, dsc, dx = _dev(nz), _dev(sg), _dev(sc), _dev(x)
    y = torch.zeros(n, dtype=torch.float16, device=DEV)
    tl.ternary_gemv(dnz, dsg, dsc, dx, y, n, k)
    q = torch.zeros(k, dtype=torch.int8, device=DEV)
    s = torch.zeros(1, dtype=torch.float32, device=DEV)
    tl.quantize_absmax_int8(dx, q, s, k)
    yi = torch.zeros(n, dtype=torch.float16, device=DEV)
    tl.ternary_gemv_int8(dnz, dsg, dsc, q, float(s.item()), yi, n, k)
    torch.cuda.synchronize()
    for out, tol in ((y, 1e-2), (yi, 5e-2)):
        err = np.abs(out.cpu().numpy().astype(np.float32) - yref)
        rel = np.where(np.abs(yref) > 1e-6, err / np.maximum(np.abs(yref), 1e-30), err)
        assert rel.max() < tol or err.max() < tol


@pytest.mark.parametrize("m,n,k", [(1, 64, 256), (3, 40, 384), (17, 128, 512), (33, 257, 1024),
                                   (128, 512, 1024)])
def test_gemm_vs_oracle(m, n, k):
    nz, sg, sc, a = oracle.make_case(n, k, seed=m * 3 + n, batch=m)
    c = torch.full((m, n), float("nan"), dtype=torch.float16, device=DEV)
    tl.ternary_gemm(_dev(a), _dev(nz), _dev(sg), _dev(sc), c, m, n, k)
    torch.cuda.synchronize()
    y64, bound = exact_and_bound(nz, sg, sc, a)
    assert_within(c.cpu().numpy(), y64, bound, f"gemm {m}x{n}x{k}", slack=_half_ulp(y64))


def test_status_codes_on_device():
    n, k = 16, 256
    nz, sg, sc, x = oracle.make_case(n, k, seed=1)
    dnz, dsg, dsc, dx = _dev(nz), _dev(sg), _dev(sc), _dev(x)
    y = torch.zeros(n, dtype=torch.float16, device=DEV)
    h, st = tl.lib(), torch.cuda.current_stream().cuda_stream
    p = [t.data_ptr() for t in (dnz, dsg, dsc, dx, y)]
    assert h.tllm_b200_gemv(*p, n, 200, 128, st) == -3
    assert h.tllm_b200_gemv(*p, n, k, 64, st) == -4
    assert h.tllm_b200_gemv_batched(*p, 17, n, k, 128, st) == -5
    with pytest.raises(ValueError):                  # the Python mirror refuses the shape before the call
        tl.ternary_gemv(dnz, dsg, dsc, dx, y, n, 200)
    with pytest.raises(tl.TllmError) as e:
        tl.ternary_gemv(dnz, dsg, dsc, dx, y, n, k, group_size=64)
    assert e.value.status == -4
    tl.ternary_gemv(dnz, dsg, dsc, dx, y, n, k)      # the context is still usable
    torch.cuda.synchronize()


@pytest.mark.skipif(not cpu.have_ref(), reason="reference kernels not built (oracle/_ref)")
def test_against_reference_cuda_kernels():
    """The reference's own kernels, compiled unmodified for sm_100, on the same inputs."""
    n, k = 1024, 4096
    nz, sg, sc, x = oracle.make_case(n, k, seed=77)
    dnz, dsg, dsc, dx = _dev(nz), _dev(sg), _dev(sc), _dev(x)
    y_ref = torch.zeros(n, dtype=torch.float16, device=DEV)
    y = torch.zeros(n, dtype=torch.float16, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    assert cpu.ref().ref_ternary_gemv(dnz.data_ptr(), dsg.data_ptr(), dsc.data_ptr(), dx.data_ptr(),
                                      y_ref.data_ptr(), n, k, 128, st) == 0
    tl.ternary_gemv(dnz, dsg, dsc, dx, y, n, k)
    torch.cuda.synchronize()
    y64, bound = exact_and_bound(nz, sg, sc, x[0])
    assert_within(y.cpu().numpy(), y64, bound, "ours", slack=_half_ulp(y64))
    assert_within(y_ref.cpu().numpy(), y64, bound, "reference kernel", slack=_half_ulp(y64))
    # quantiser: bit-exact against the reference kernel
    q_ref = torch.zeros(k, dtype=torch.int8, device=DEV)
    q = torch.zeros(k, dtype=torch.int8, device=DEV)
    s_ref = torch.zeros(1, dtype=torch.float32, device=DEV)
    s = torch.zeros(1, dtype=torch.float32, device=DEV)
    assert cpu.ref().ref_quantize_absmax_int8(dx.data_ptr(), q_ref.data_ptr(), s_ref.data_ptr(), k, st) == 0
    tl.quantize_absmax_int8(dx, q, s, k)
    torch.cuda.synchronize()
    # the reference build uses --use_fast_math, so its reciprocal may differ in the last
    # ulp: allow values that sit on a rounding boundary to differ by one step
    d = (q.cpu().numpy().astype(np.int32) - q_ref.cpu().numpy().astype(np.int32))
    assert np.abs(d).max() <= 1 and (d != 0).mean() < 1e-3
    assert abs(s.item() - s_ref.item()) <= 2.4e-7 * abs(s.item())   # fast-math division: 1-2 ulp
    # GEMM against the reference GEMM kernel
    m = 8
    a = np.random.default_rng(3).standard_normal((m, k)).astype(np.float16)
    da = _dev(a)
    c_ref = torch.zeros(m, n, dtype=torch.float16, device=DEV)
    c = torch.zeros(m, n, dtype=torch.float16, device=DEV)
    assert cpu.ref().ref_ternary_gemm(da.data_ptr(), dnz.data_ptr(), dsg.data_ptr(), dsc.data_ptr(),
                                      c_ref.data_ptr(), m, n, k, 128, st) == 0
    tl.ternary_gemm(da, dnz, dsg, dsc, c, m, n, k)
    torch.cuda.synchronize()
    y64, bound = exact_and_bound(nz, sg, sc, a)
    assert_within(c.cpu().numpy(), y64, bound, "gemm ours", slack=_half_ulp(y64))
    assert_within(c_ref.cpu().numpy(), y64, bound, "gemm reference kernel", slack=_half_ulp(y64))
