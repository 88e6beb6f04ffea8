"""Drop-in proof: the reference's own sources, unmodified, against libtllm_b200.so.

oracle/Makefile target `dropin` links (a) the reference's GPU test
tests/test_ternary_gemv.cu and (b) its engine sources src/transformer.cpp +
src/model.cpp (+ its other kernels) against this library in place of
kernels/ternary_gemv.cu, kernels/ternary_gemm.cu and the quantiser.  The CPU test
checks that the operator symbols those binaries need are the ones the library
exports; the GPU test runs the reference's test binary."""
import os
import subprocess

import pytest

import ternary_llm_b200 as tl
from oracle import cpu

NEEDED = ["_ZN7ternary12ternary_gemvEPKjS1_PK6__halfS4_PS2_iiiP11CUstream_st",
          "_ZN7ternary17ternary_gemv_int8EPKjS1_PK6__halfPKafPS2_iiiP11CUstream_st",
          "_ZN7ternary20quantize_absmax_int8EPK6__halfPaPfiP11CUstream_st",
          "_ZN7ternary12ternary_gemmEPK6__halfPKjS4_S2_PS0_iiiiP11CUstream_st"]


def _nm(path, flag):
    out = subprocess.run(["nm", "-D", flag, path], capture_output=True, text=True, check=True).stdout
    return {line.split()[-1] for line in out.splitlines() if line.strip()}


def test_library_exports_the_reference_operator_symbols():
    exported = _nm(tl.LIB_PATH, "--defined-only")
    for sym in NEEDED:
        assert sym in exported, sym


@pytest.mark.skipif(not (os.path.exists(cpu.DROPIN_TEST) and os.path.exists(cpu.ENGINE_LINK)),
                    reason="drop-in binaries not built (needs the reference checkout)")
def test_reference_binaries_take_the_operators_from_the_library():
    test_needs = _nm(cpu.DROPIN_TEST, "--undefined-only")
    assert set(NEEDED[:3]) <= test_needs            # gemv, gemv_int8, quantiser come from the library
    engine_needs = _nm(cpu.ENGINE_LINK, "--undefined-only")
    assert {NEEDED[0], NEEDED[1], NEEDED[3]} <= engine_needs   # transformer.cpp's gemv / gemv_int8 / gemm


@pytest.mark.gpu
@pytest.mark.skipif(not os.path.exists(cpu.DROPIN_TEST), reason="drop-in test binary not built")
def test_reference_gpu_test_passes_on_this_library():
    r = subprocess.run([cpu.DROPIN_TEST], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "6 / 6 tests passed" in r.stdout
