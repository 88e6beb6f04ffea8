#!/usr/bin/env python3
"""Times the REFERENCE's own CUDA kernels (compiled unmodified for sm_100 into
oracle/_ref/libref.so) on a B200, on seeded non-zero weights, as a reported baseline
beside this library's kernels.  Not a pytest module; run by hand on a GPU machine:

    python tests/time_reference_kernels.py

Cold weights: each timed launch uses a different matrix (working set > L2)."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import ternary_llm_b200 as tl  # noqa: E402
from oracle import cpu  # noqa: E402
from ternary_llm_b200 import synth  # noqa: E402


def timed(fn, n_launch, reps=3):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * n_launch)


def main():
    dev = torch.device("cuda", 0)
    ref = cpu.ref()
    st = torch.cuda.current_stream().cuda_stream
    for name, n, k in (("q/o 4096x4096", 4096, 4096), ("gate/up 14336x4096", 14336, 4096), ("down 4096x14336", 4096, 14336)):
        copies = 12
        ws = [synth.random_ternary_weight(n, k, seed=i, device=dev) for i in range(copies)]
        prep = [tl.PreparedWeight(a, b, c, n, k, register=False) for a, b, c in ws]
        x = torch.randn(k, device=dev).half()
        xq = torch.randint(-127, 128, (k,), device=dev, dtype=torch.int8)
        y = torch.zeros(n, device=dev, dtype=torch.float16)
        nbytes = n * k // 4 + n * k // 64 + 2 * (n + k)

        def ref_gemv():
            for a, b, c in ws:
                ref.ref_ternary_gemv(a.data_ptr(), b.data_ptr(), c.data_ptr(), x.data_ptr(), y.data_ptr(), n, k, 128, st)

        def ref_gemv_int8():
            for a, b, c in ws:
                ref.ref_ternary_gemv_int8(a.data_ptr(), b.data_ptr(), c.data_ptr(), xq.data_ptr(), 0.01, y.data_ptr(), n, k, 128, st)

        def ours():
            for w in prep:
                tl.ternary_gemv_packed(w, x, y, 1)

        for label, fn in (("reference ternary_gemv", ref_gemv), ("reference ternary_gemv_int8", ref_gemv_int8),
                          ("this library (stream launches)", ours)):
            us = timed(fn, copies)
            print(f"{name:22s} {label:32s} {us:9.2f} us  {nbytes / us / 1e3:8.1f} GB/s")
        m = 128
        a_act = torch.randn(m, k, device=dev).half()
        c_out = torch.zeros(m, n, device=dev, dtype=torch.float16)
        a, b, c = ws[0]
        us = timed(lambda: ref.ref_ternary_gemm(a_act.data_ptr(), a.data_ptr(), b.data_ptr(), c.data_ptr(),
                                                c_out.data_ptr(), m, n, k, 128, st), 1)
        print(f"{name:22s} {'reference ternary_gemm M=128':32s} {us:9.2f} us  {2 * m * n * k / us / 1e6:8.2f} TFLOP/s")
        us = timed(lambda: tl.ternary_gemm_packed(a_act, prep[0], c_out, m), 1)
        print(f"{name:22s} {'this library gemm M=128':32s} {us:9.2f} us  {2 * m * n * k / us / 1e6:8.2f} TFLOP/s")


if __name__ == "__main__":
    main()
