"""Size-independent properties of the packing, the oracle and the host-side sharding, on
randomly drawn shapes (hypothesis): pack <-> unpack round trips, the product packer agrees
with the oracle's, linearity of the contraction, quantiser bounds, shards reassemble."""
import numpy as np
from hypothesis import given, settings, strategies as st

from oracle import oracle
from ternary_llm_b200 import pack
from ternary_llm_b200 import tllm_format as tf

SETTINGS = dict(max_examples=25, deadline=None)


def _ternary(rng, n, k, p_zero):
    t = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
    t[rng.random((n, k)) < p_zero] = 0
    return t


@settings(**SETTINGS)
@given(n=st.integers(1, 40), words=st.integers(1, 12), p=st.floats(0.0, 1.0), seed=st.integers(0, 2 ** 31 - 1))
def test_pack_unpack_round_trip_and_packers_agree(n, words, p, seed):
    rng = np.random.default_rng(seed)
    t = _ternary(rng, n, 32 * words, p)
    nz, sg = pack.pack_ternary_to_bitmasks(t)
    nz_o, sg_o = oracle.pack_ternary_to_bitmasks(t)
    assert nz.dtype == np.uint32 and nz.shape == (n, words)
    assert np.array_equal(nz, nz_o) and np.array_equal(sg, sg_o)
    assert not (sg & ~nz).any()                                  # canonical: sign bits only under nonzero bits
    assert np.array_equal(pack.unpack_bitmasks(nz, sg), t)
    assert np.array_equal(oracle.unpack_bitmasks(nz, sg), t)


@settings(**SETTINGS)
@given(n=st.integers(1, 24), groups=st.integers(1, 4), seed=st.integers(0, 2 ** 31 - 1))
def test_contraction_is_linear_in_the_activations(n, groups, seed):
    k = 128 * groups
    nz, sg, sc, x = oracle.make_case(n, k, seed=seed, batch=2)
    x1, x2 = x[0].astype(np.float64), x[1].astype(np.float64)
    w = oracle.dequantize(nz, sg, sc).astype(np.float64)
    y1 = oracle.ternary_matvec(nz, sg, sc, x[0], 128, np.float64)
    y2 = oracle.ternary_matvec(nz, sg, sc, x[1], 128, np.float64)
    assert np.allclose(w @ (x1 + x2), y1 + y2, rtol=1e-12, atol=1e-12)
    # the GEMM oracle is the matvec per token
    c = oracle.ternary_gemm(x, nz, sg, sc)
    assert c.shape == (2, n)


@settings(**SETTINGS)
@given(n=st.integers(1, 300), scale=st.floats(1e-3, 1e3), seed=st.integers(0, 2 ** 31 - 1))
def test_quantiser_bounds(n, scale, seed):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(n) * scale).astype(np.float16)
    q, s = oracle.quantize_absmax_int8(x)
    assert q.dtype == np.int8 and np.abs(q.astype(np.int32)).max() <= 127
    xf = x.astype(np.float32)
    amax = float(np.abs(xf).max())
    if amax == 0.0:
        assert s == 1.0 and not q.any()
    else:
        assert np.isclose(s, amax / 127.0, rtol=1e-6)
        assert (np.abs(q.astype(np.float32) * s - xf) <= 0.5 * s * (1 + 1e-5) + 1e-12).all()
        assert np.abs(q.astype(np.int32)).max() == 127                     # the largest element maps to +-127


@settings(**SETTINGS)
@given(world=st.sampled_from([1, 2, 4]), rows_per=st.integers(1, 6), groups_per=st.integers(1, 2),
       seed=st.integers(0, 2 ** 31 - 1))
def test_shards_tile_the_matrix(world, rows_per, groups_per, seed):
    n, k = rows_per * world, groups_per * world * 128
    nz, sg, sc, _ = oracle.make_case(n, k, seed=seed)
    t = tf.TernaryTensor(nz, sg, sc)
    cols = [tf.shard_ternary(t, "gate_proj", r, world) for r in range(world)]
    assert np.array_equal(np.concatenate([c.nonzero_masks for c in cols], 0), nz)
    assert np.array_equal(np.concatenate([c.scales for c in cols], 0).view(np.uint16), sc.view(np.uint16))
    rows = [tf.shard_ternary(t, "down_proj", r, world) for r in range(world)]
    assert np.array_equal(np.concatenate([c.sign_masks for c in rows], 1), sg)
    assert np.array_equal(np.concatenate([c.scales for c in rows], 1).view(np.uint16), sc.view(np.uint16))
    assert all(c.shape == (n, k // world) for c in rows)
