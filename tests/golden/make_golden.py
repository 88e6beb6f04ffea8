#!/usr/bin/env python3
"""Regenerate the golden fixtures from the reference project itself.

Needs a checkout of jastaq/ternary-llm (--ref, default oracle.cpu.REF_DIR) and
oracle/_ref/libref.so (make -C oracle ref).  It imports the reference's own
ternarize/pack.py for the packing fixtures and calls the reference's compiled
cpu_reference (tests/test_ternary_gemv.cu:40-75) for the matvec fixtures, so the
stored outputs come from the reference's code, not from this repository's
restatement.  The fixtures are small .npz files committed beside this script.

    python tests/golden/make_golden.py [--ref /path/to/reference]
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def main():
    from oracle.cpu import REF_DIR
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=REF_DIR)
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.ref, "ternarize"))
    sys.path.insert(0, os.path.join(args.ref, "tests"))
    import pack as refpack                      # the reference's packer
    from test_packing import unpack_bitmasks    # the reference's unpacker (triple loop)
    from oracle import cpu

    # ---- packing fixtures -------------------------------------------------
    out = {}
    cases = []
    # (name, weight tensor) -- the first two repeat the reference's seeded tests
    torch.manual_seed(123)                      # tests/test_packing.py:145
    cases.append(("seed123_64x100", refpack.pad_to_multiple(torch.randn(64, 100), 32)))
    torch.manual_seed(42)                       # tests/test_packing.py:96
    cases.append(("seed42_256x128", torch.randn(256, 128)))
    g = torch.Generator().manual_seed(7)
    cases.append(("w002_24x512", 0.02 * torch.randn(24, 512, generator=g)))
    w = 0.02 * torch.randn(8, 256, generator=g)
    w[3, :128] = 0.0                            # an all-zero group -> scale 0
    w[5, 128:] = 100.0 * torch.sign(w[5, 128:])  # large values -> all nonzero
    cases.append(("edge_8x256", w))
    for name, wt in cases:
        tern, scales = refpack.ternarize_tensor(wt, group_size=128, threshold_factor=0.7)
        nz, sg = refpack.pack_ternary_to_bitmasks(tern)
        assert (unpack_bitmasks(nz, sg) == tern.numpy()).all()
        out[name + "/w"] = wt.numpy().astype(np.float32)
        out[name + "/ternary"] = tern.numpy()
        out[name + "/scales"] = scales.numpy()
        out[name + "/nz"] = nz
        out[name + "/sign"] = sg
    np.savez_compressed(os.path.join(HERE, "packing.npz"), **out)

    # ---- matvec fixtures: outputs of the reference's cpu_reference ----------
    out = {}
    rng = np.random.default_rng(20261125)
    specs = [("rand_9x128", 9, 128, True), ("rand_16x256", 16, 256, True),
             ("rand_64x1024", 64, 1024, True), ("tern_48x2048", 48, 2048, False),
             ("tern_128x512", 128, 512, False)]
    for name, n, k, random_masks in specs:
        if random_masks:   # independent random words, signed scales: tests/test_ternary_gemv.cu:98-108
            nz = rng.integers(0, 2**32, size=(n, k // 32), dtype=np.uint64).astype(np.uint32)
            sg = rng.integers(0, 2**32, size=(n, k // 32), dtype=np.uint64).astype(np.uint32)
            sc = rng.uniform(-0.1, 0.1, size=(n, k // 128)).astype(np.float16)
        else:
            wt = torch.from_numpy((0.02 * rng.standard_normal((n, k))).astype(np.float32))
            tern, scales = refpack.ternarize_tensor(wt, 128, 0.7)
            nz, sg = refpack.pack_ternary_to_bitmasks(tern)
            sc = scales.numpy().reshape(n, k // 128)
        x = rng.standard_normal(k).astype(np.float16)
        y = cpu.matvec_f32(nz, sg, sc.astype(np.float32), x.astype(np.float32), 128, use_ref=True)
        out[name + "/nz"], out[name + "/sign"] = nz, sg
        out[name + "/scales"], out[name + "/x"], out[name + "/y"] = sc, x, y
    np.savez_compressed(os.path.join(HERE, "matvec.npz"), **out)
    print("wrote", os.path.join(HERE, "packing.npz"), os.path.join(HERE, "matvec.npz"))


if __name__ == "__main__":
    main()
