"""GPU parity tests of the tcgen05 prefill GEMM on prepared weights."""
import numpy as np
import pytest
import torch

import ternary_llm_b200 as tl
from oracle import oracle
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


def _gemm(nz, sg, sc, a, registered=False):
    n, k = nz.shape[0], nz.shape[1] * 32
    m = a.shape[0]
    dnz, dsg, dsc = _dev(nz), _dev(sg), _dev(sc)
    w = tl.PreparedWeight(dnz, dsg, dsc, n, k, register=registered)
    c = torch.full((m, n), float("nan"), dtype=torch.float16, device=DEV)
    if registered:
        tl.ternary_gemm(_dev(a), dnz, dsg, dsc, c, m, n, k)     # the reference-signature call
    else:
        tl.ternary_gemm_packed(_dev(a), w, c, m)
    torch.cuda.synchronize()
    tl.check_device_errors()
    w.release()
    return c.cpu().numpy()


@pytest.mark.parametrize("m,n,k", [(17, 128, 128), (32, 128, 256), (64, 256, 512), (128, 512, 1024),
                                   (200, 200, 384), (257, 129, 640), (300, 1000, 2048), (512, 1024, 4096)])
def test_gemm_tcgen05_vs_oracle(m, n, k):
    nz, sg, sc, a = oracle.make_case(n, k, seed=m + 2 * n + k, batch=m)
    c = _gemm(nz, sg, sc, a)
    y64, bound = exact_and_bound(nz, sg, sc, a)
    assert not np.isnan(c).any()
    assert_within(c, y64, bound, f"gemm {m}x{n}x{k}", slack=_half_ulp(y64))


def test_gemm_signed_scales_and_edge_rows():
    m, n, k = 96, 160, 512
    nz, sg, sc, a = oracle.make_case(n, k, seed=5, batch=m, random_masks=True, signed_scales=True)
    sg &= nz
    nz[3], sg[3] = 0, 0
    sc[4] = 0
    nz[6], sg[6] = 0xFFFFFFFF, 0xFFFFFFFF
    nz[7], sg[7] = 0xFFFFFFFF, 0
    c = _gemm(nz, sg, sc, a)
    y64, bound = exact_and_bound(nz, sg, sc, a)
    assert (c[:, 3] == 0).all() and (c[:, 4] == 0).all()
    assert_within(c, y64, bound, "gemm edge", slack=_half_ulp(y64))


def test_gemm_through_reference_signature():
    m, n, k = 130, 384, 1024
    nz, sg, sc, a = oracle.make_case(n, k, seed=31, batch=m)
    c = _gemm(nz, sg, sc, a, registered=True)
    y64, bound = exact_and_bound(nz, sg, sc, a)
    assert_within(c, y64, bound, "gemm registered", slack=_half_ulp(y64))


def test_gemm_full_size_against_gemv_and_sampled_oracle():
    """M=2048 at a LLaMA-3-8B shape: sampled tokens against the oracle, and three token
    blocks against the GEMV kernel on the same prepared weights."""
    m, n, k = 2048, 4096, 4096
    nz, sg, sc = tl.pack.random_ternary_weight(n, k, seed=12)
    a = np.random.default_rng(13).standard_normal((m, k)).astype(np.float16)
    dnz, dsg, dsc, da = _dev(nz), _dev(sg), _dev(sc), _dev(a)
    w = tl.PreparedWeight(dnz, dsg, dsc, n, k, register=False)
    c = torch.full((m, n), float("nan"), dtype=torch.float16, device=DEV)
    tl.ternary_gemm_packed(da, w, c, m)
    torch.cuda.synchronize()
    tl.check_device_errors()
    rows = np.random.default_rng(1).choice(m, 24, replace=False)
    y64, bound = exact_and_bound(nz, sg, sc, a[rows])
    assert_within(c.cpu().numpy()[rows], y64, bound, "gemm 2048 sampled", slack=_half_ulp(y64))
    # every output of three token blocks against the streaming GEMV (four vectors per pass: the
    # mma.sync kernel, which shares no code with the tcgen05 one) on the same prepared weights
    for m0 in (0, 1008, 2044):
        y = torch.zeros(4, n, dtype=torch.float16, device=DEV)
        tl.ternary_gemv_packed(w, da[m0:m0 + 4], y, 4)
        torch.cuda.synchronize()
        d = (y.float() - c[m0:m0 + 4].float()).abs().cpu().numpy()
        ref = np.abs(y.float().cpu().numpy())
        assert (d <= ref * 2.0 ** -9 + 2e-3).all()
