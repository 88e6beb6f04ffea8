"""Where a GEMV launch spends its time inside a stream of dependent launches.

    python -m ternary_llm_b200.build --timeline          # builds libtllm_b200_timeline.so
    python -m ternary_llm_b200.timeline 14336+14336x4096 [copies] [f16|i8]

Runs a CUDA-graph chain of GEMV launches over `copies` distinct matrices (or groups of
matrices packed back to back: N1+N2xK) on the diagnostic build of the library, whose GEMV
kernel records the GPU nanosecond timer at seven points per CTA, and prints the medians over
the CTAs: kernel entry, first ring fill issued, stream-order wait over, activations staged,
last tile done, partial sums exchanged inside the CTA, outputs written.  The shipped library
records nothing; this module refuses to run on it.
"""
from __future__ import annotations

import ctypes
import os
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
NAMES = ["entry", "fill issued", "wait over", "x staged", "tiles done", "cta sums", "outputs"]


def main(argv) -> int:
    if not argv:
        print(__doc__)
        return 2
    lib = os.path.join(PKG, "libtllm_b200_timeline.so")
    if not os.path.exists(lib):
        print("build the diagnostic library first: python -m ternary_llm_b200.build --timeline", file=sys.stderr)
        return 1
    import numpy as np
    import torch

    import ternary_llm_b200 as tl
    from ternary_llm_b200 import _lib, synth
    _lib.LIB_PATH = lib                        # the library is loaded on first use: not yet

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    ns, k = argv[0].split("x")
    shapes, k = [int(v) for v in ns.split("+")], int(k)
    copies = int(argv[1]) if len(argv) > 1 else 8
    mode = argv[2] if len(argv) > 2 else "f16"
    sets = []
    for c in range(copies):
        sets.append(tl.prepare_group([synth.random_ternary_weight(n, k, seed=c * 10 + i, device=dev) + (n, k)
                                      for i, n in enumerate(shapes)]))
    x = torch.randn(k, device=dev).half()
    xq = torch.randint(-127, 127, (k,), device=dev, dtype=torch.int8)
    ys = [torch.zeros(n, device=dev, dtype=torch.float16) for n in shapes]

    def go():
        for ws in sets:
            if mode == "i8":
                tl.ternary_gemv_int8_packed(ws[0], xq, 0.01, ys[0])
            elif len(ws) > 1:
                tl.ternary_gemv_packed_multi(ws, x, ys)
            else:
                tl.ternary_gemv_packed(ws[0], x, ys[0], 1)

    go()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            go()
        for _ in range(4):
            g.replay()
        torch.cuda.synchronize()
    h = tl.lib()
    if not hasattr(h, "tllm_b200_timeline_read"):
        print("the loaded library has no time stamps (not the diagnostic build)", file=sys.stderr)
        return 1
    buf = np.zeros((8, 256, 8), np.uint64)
    cnt = np.zeros(256, np.uint32)
    h.tllm_b200_timeline_read.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    if h.tllm_b200_timeline_read(buf.ctypes.data, cnt.ctypes.data) != 0:
        return 1
    ctas = np.nonzero(cnt == cnt.max())[0]
    last = int(cnt.max()) - 1
    info = int(buf[last & 7, ctas[0], 7])
    print(f"{argv[0]} {mode}: grid {(info >> 20) & 4095}, whole row blocks per CTA: {info & 255}, "
          f"ring slots {(info >> 8) & 4095}; medians over {len(ctas)} CTAs, microseconds")
    t_ref = None
    for back in (2, 1, 0):
        rec = buf[(last - back) & 7][ctas][:, :7].astype(np.int64)
        if t_ref is None:
            t_ref = rec[:, 0].min()
        r = (rec - t_ref) / 1e3
        print(f" launch -{back}: " + "  ".join(f"{nm} {np.median(r[:, i]):6.2f}" for i, nm in enumerate(NAMES)))
        d = np.diff(r, axis=1)
        print("   phase lengths: " + "  ".join(f"{np.median(d[:, i]):5.2f}" for i in range(6)))
    out = [np.median(buf[(last - b) & 7][ctas][:, 6].astype(np.int64)) for b in (3, 2, 1, 0)]
    print(" period between launches: " + ", ".join(f"{(out[i + 1] - out[i]) / 1e3:.2f}" for i in range(3)) + " us")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
