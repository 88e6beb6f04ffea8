"""The oracle against the reference's known answers and the golden fixtures.

CPU only.  Pins oracle/oracle.py and oracle/cpu_reference.c to
  * the explicit words of the reference's packing test (tests/test_packing.py:48-89),
  * packing.npz: outputs of the reference's ternarize/pack.py,
  * matvec.npz: outputs of the reference's compiled cpu_reference.
"""
import os

import numpy as np
import pytest

from oracle import cpu, oracle


def _load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name))
    cases = {}
    for key in z.files:
        case, field = key.split("/")
        cases.setdefault(case, {})[field] = z[key]
    return cases


def test_known_answer_words():
    # tests/test_packing.py:52-81
    t = np.zeros((2, 64), np.int8)
    t[0, 0], t[0, 1], t[0, 31], t[0, 32], t[0, 63] = 1, -1, 1, -1, -1
    t[1, :32] = np.where(np.arange(32) % 2 == 0, 1, -1)
    nz, sg = oracle.pack_ternary_to_bitmasks(t)
    assert nz.shape == (2, 2) and nz.dtype == np.uint32
    assert nz[0, 0] == 0x80000003 and sg[0, 0] == 0x80000001
    assert nz[0, 1] == 0x80000001 and sg[0, 1] == 0
    assert nz[1, 0] == 0xFFFFFFFF and sg[1, 0] == 0x55555555
    assert (oracle.unpack_bitmasks(nz, sg) == t).all()
    assert (oracle.unpack_bitmasks_loop(nz, sg) == t).all()


def test_noncanonical_sign_bits_decode_to_zero():
    nz = np.array([[0x0000000F]], np.uint32)
    sg = np.array([[0xFFFFFFF5]], np.uint32)
    t = oracle.unpack_bitmasks(nz, sg)
    assert t[0, :4].tolist() == [1, -1, 1, -1] and (t[0, 4:] == 0).all()


def test_vectorised_unpack_equals_loop():
    rng = np.random.default_rng(0)
    nz = rng.integers(0, 2**32, (5, 3), dtype=np.uint64).astype(np.uint32)
    sg = rng.integers(0, 2**32, (5, 3), dtype=np.uint64).astype(np.uint32)
    assert (oracle.unpack_bitmasks(nz, sg) == oracle.unpack_bitmasks_loop(nz, sg)).all()


def test_packing_fixtures(golden_dir):
    for name, c in _load(golden_dir, "packing.npz").items():
        tern, scales = oracle.ternarize_tensor(c["w"], 128, 0.7)
        assert (tern == c["ternary"]).all(), name
        assert (scales.view(np.uint16) == c["scales"].view(np.uint16)).all(), name
        nz, sg = oracle.pack_ternary_to_bitmasks(c["ternary"])
        assert (nz == c["nz"]).all() and (sg == c["sign"]).all(), name
        assert (oracle.unpack_bitmasks(c["nz"], c["sign"]) == c["ternary"]).all(), name
        assert (c["sign"] & ~c["nz"] == 0).all(), name


def test_edge_fixture_semantics(golden_dir):
    c = _load(golden_dir, "packing.npz")["edge_8x256"]
    sc = c["scales"].reshape(8, 2)
    assert sc[3, 0] == 0 and (c["ternary"][3, :128] == 0).all()       # tests/test_packing.py:177-186
    assert (c["ternary"][5, 128:] != 0).all()                           # tests/test_packing.py:189-205


def test_pad_to_multiple():
    w = np.ones((4, 50), np.float32)
    p = oracle.pad_to_multiple(w, 32)
    assert p.shape == (4, 64) and (p[:, :50] == 1).all() and (p[:, 50:] == 0).all()
    assert oracle.pad_to_multiple(p, 32) is p
    assert oracle.pad_to_multiple(np.ones(100, np.float32), 32).shape == (128,)


def test_matvec_fixtures_numpy(golden_dir):
    for name, c in _load(golden_dir, "matvec.npz").items():
        y64 = oracle.ternary_matvec(c["nz"], c["sign"], c["scales"], c["x"], 128, np.float64)
        tol = oracle.tolerance_bound(c["nz"], c["sign"], c["scales"], c["x"])
        # the reference's float32 result agrees with the exact value far inside the bound
        assert (np.abs(c["y"] - y64) <= 0.02 * tol + 1e-12).all(), name
        y32 = oracle.ternary_matvec(c["nz"], c["sign"], c["scales"], c["x"], 128, np.float32)
        assert (np.abs(y32 - y64) <= 0.02 * tol + 1e-12).all(), name


def test_matvec_fixtures_c_port_bit_exact(golden_dir):
    # same scalar order of operations as the reference -> identical float32 bits
    for name, c in _load(golden_dir, "matvec.npz").items():
        y = cpu.matvec_f32(c["nz"], c["sign"], c["scales"].astype(np.float32),
                           c["x"].astype(np.float32), 128)
        assert (y.view(np.uint32) == c["y"].view(np.uint32)).all(), name
        ymt = cpu.matvec_f32(c["nz"], c["sign"], c["scales"].astype(np.float32),
                             c["x"].astype(np.float32), 128, threads=2)
        assert (ymt.view(np.uint32) == c["y"].view(np.uint32)).all(), name
        yh = cpu.matvec_f16(c["nz"], c["sign"], c["scales"], c["x"], 128, threads=2)
        assert (yh.view(np.uint32) == c["y"].view(np.uint32)).all(), name


@pytest.mark.skipif(not cpu.have_ref(), reason="oracle/_ref not built on this machine")
def test_c_port_equals_compiled_reference():
    nz, sg, sc, x = oracle.make_case(37, 384, seed=5, random_masks=True, signed_scales=True)
    a = cpu.matvec_f32(nz, sg, sc.astype(np.float32), x[0].astype(np.float32), use_ref=True)
    b = cpu.matvec_f32(nz, sg, sc.astype(np.float32), x[0].astype(np.float32))
    c = cpu.matvec_f32(nz, sg, sc.astype(np.float32), x[0].astype(np.float32), use_ref=True, threads=3)
    assert (a.view(np.uint32) == b.view(np.uint32)).all()
    assert (a.view(np.uint32) == c.view(np.uint32)).all()


def test_quantize_absmax_int8_semantics():
    # kernels/activations.cu:88-142
    q, s = oracle.quantize_absmax_int8(np.zeros(16, np.float16))
    assert s == 1.0 and (q == 0).all()
    x = np.array([2.0, -2.0, 1.0, 0.5 * 2 / 127, 1.5 * 2 / 127, 2.5 * 2 / 127], np.float32).astype(np.float16)
    q, s = oracle.quantize_absmax_int8(x)
    assert q[0] == 127 and q[1] == -127 and np.isclose(s, 2.0 / 127)
    xf = x.astype(np.float32)
    inv = np.float32(127.0) / np.float32(2.0)
    assert (q == np.clip(np.rint(xf * inv), -127, 127)).all()
    assert np.rint(np.float32(0.5)) == 0 and np.rint(np.float32(1.5)) == 2   # ties to even


def test_int8_matvec_consistency():
    nz, sg, sc, x = oracle.make_case(33, 256, seed=3)
    q, s = oracle.quantize_absmax_int8(x[0])
    y = oracle.ternary_matvec_int8(nz, sg, sc, q, s)
    yc = cpu.matvec_i8(nz, sg, sc, q, s, threads=2)
    y64 = oracle.ternary_matvec(nz, sg, sc, q.astype(np.float64) * np.float64(s), 128, np.float64)
    tol = oracle.tolerance_bound_int8(nz, sg, sc, q, s)
    assert (np.abs(y - y64) <= 0.02 * tol).all()
    assert (np.abs(yc - y64) <= 0.02 * tol).all()


def test_gemm_oracle_is_batched_matvec():
    nz, sg, sc, a = oracle.make_case(20, 256, seed=9, batch=5)
    c = oracle.ternary_gemm(a, nz, sg, sc)
    w = oracle.dequantize(nz, sg, sc)
    assert np.allclose(c, a.astype(np.float32) @ w.T, rtol=1e-4, atol=1e-5)
    yc = cpu.matvec_f16(nz, sg, sc, a, threads=2)
    assert np.allclose(c, yc, rtol=1e-4, atol=1e-5)


def test_make_case_distribution():
    nz, sg, sc, x = oracle.make_case(256, 2048, seed=0)
    t = oracle.unpack_bitmasks(nz, sg)
    z = (t == 0).mean()
    assert 0.40 < z < 0.44 and abs((t == 1).mean() - (t == -1).mean()) < 0.01
    assert 0.017 < float(sc.astype(np.float32).mean()) < 0.031
