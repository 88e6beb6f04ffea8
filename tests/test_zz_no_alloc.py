"""The allocation-free GEMV entry point against the regular one.

tllm_b200_gemv_packed_noalloc exists for hosts that cannot allow a library to call
cudaMalloc (their own arena owns the device memory, or allocation is forbidden where
the call is made); its split-K scratch is a fixed array inside the library.  This
test calls it straight through the C ABI, twice in a row on each shape, and compares
with tllm_b200_gemv_packed on the same prepared weights.  The two may add the K
groups in a different order, so they are compared to within one FP16 last place and
each against the oracle with the 2e-3 * sum|scale*x| tolerance the other tests use;
the two calls in a row must agree exactly with each other, which checks that the
shared scratch is left reusable, and the amount of free device memory must be the same
before and after them.  tllm_b200_gemv_packed_noalloc_status is the allocation-free way
to learn that a bounded wait expired; it must report none.
The file name sorts last so that a stop-at-first-failure run has already executed
every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

import ternary_llm_b200 as tl
from ternary_llm_b200 import _lib
from oracle import oracle
from tests._util import assert_within, exact_and_bound

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _dev(a):
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).to(DEV)
    return torch.from_numpy(a).to(DEV)


# (1024, 4096) splits K across SMs, so the scratch records and counters are exercised;
# (4096, 4096) takes whole row blocks per CTA; (40, 384) has ragged rows.
@pytest.mark.parametrize("n,k", [(1024, 4096), (4096, 4096), (40, 384)])
def test_noalloc_matches_regular_entry_point_twice(n, k):
    torch.cuda.set_device(0)
    nz, sg, sc, x = oracle.make_case(n, k, seed=n + k + 1)
    w = tl.PreparedWeight(_dev(nz), _dev(sg), _dev(sc), n, k, register=False)
    dx = _dev(x[0])
    h = tl.lib()
    stream = torch.cuda.current_stream().cuda_stream

    y_ref = torch.full((n,), float("nan"), dtype=torch.float16, device=DEV)
    _lib.check(h.tllm_b200_gemv_packed(w.packed.data_ptr(), dx.data_ptr(), y_ref.data_ptr(), 1, n, k, stream))

    # one call first, so that the one-time set-up (module load, symbol lookup) is behind us; then
    # the property the entry point exists for: the two calls change nothing about device memory
    warm = torch.empty(n, dtype=torch.float16, device=DEV)
    _lib.check(h.tllm_b200_gemv_packed_noalloc(w.packed.data_ptr(), dx.data_ptr(), warm.data_ptr(), n, k, stream))
    outs = [torch.full((n,), float("nan"), dtype=torch.float16, device=DEV) for _ in range(2)]
    torch.cuda.synchronize()
    free_before, reserved_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_reserved()
    for y in outs:
        _lib.check(h.tllm_b200_gemv_packed_noalloc(w.packed.data_ptr(), dx.data_ptr(), y.data_ptr(), n, k, stream))
    assert h.tllm_b200_gemv_packed_noalloc_status(stream) == 0      # synchronises; no wait expired
    assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_reserved() == reserved_before
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])
    for y in outs:
        assert not torch.isnan(y).any()
        d = (y.float() - y_ref.float()).abs()
        assert bool((d <= y_ref.float().abs() * 2.0 ** -10 + 1e-6).all())
    y64, bound = exact_and_bound(nz, sg, sc, x[0])
    half_ulp = 0.5 * 2.0 ** (np.floor(np.log2(np.maximum(np.abs(y64), 2.0 ** -14))) - 10)
    assert_within(outs[1].cpu().numpy(), y64, bound, f"noalloc {n}x{k}", slack=half_ulp)


def test_noalloc_rejects_sizes_over_its_maximum():
    torch.cuda.set_device(0)
    h = tl.lib()
    buf = torch.zeros(4096, dtype=torch.uint8, device=DEV)
    st = h.tllm_b200_gemv_packed_noalloc(buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), 65536 + 16, 128, None)
    assert st == -9
    assert b"maximum" in h.tllm_b200_last_error()
