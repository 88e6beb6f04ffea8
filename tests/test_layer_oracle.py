"""CPU checks of the layer-operator oracle (oracle/layer_oracle.py): each restatement
against an independent float64 formulation, and the invariants of the forward pass."""
import numpy as np

from oracle import layer_oracle as LO
from ternary_llm_b200 import tllm_format as tf

f16 = np.float16


def test_rmsnorm_against_float64_and_residual_forms():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 256)).astype(f16)
    r = rng.standard_normal((3, 256)).astype(f16)
    w = (1 + 0.1 * rng.standard_normal(256)).astype(f16)
    out, ro = LO.rmsnorm(x, w, 1e-5)
    assert ro is None
    x64 = x.astype(np.float64)
    want = x64 / np.sqrt((x64 ** 2).mean(-1, keepdims=True) + 1e-5) * w.astype(np.float64)
    assert np.abs(out.astype(np.float64) - want).max() <= 2e-3 * np.abs(want).max()
    out2, ro2 = LO.rmsnorm(x, w, 1e-5, residual=r)
    assert (ro2 == (x.astype(np.float32) + r.astype(np.float32)).astype(f16)).all()
    # add-then-normalise (round_first) equals normalising the stored sum
    out3, ro3 = LO.rmsnorm(x, w, 1e-5, residual=r, round_first=True)
    out4, _ = LO.rmsnorm(ro3, w, 1e-5)
    assert (out3 == out4).all() and (ro3 == ro2).all()


def test_rope_is_a_rotation_of_interleaved_pairs():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((1, 5, 3, 64)).astype(f16)
    y = LO.rope(x, start_pos=7, theta=500000.0)
    z = x[..., 0::2].astype(np.float64) + 1j * x[..., 1::2].astype(np.float64)
    i = np.arange(32)
    ang = (7 + np.arange(5))[:, None] / (500000.0 ** (2 * i / 64))[None, :]
    zr = z * np.exp(1j * ang)[None, :, None, :]
    assert np.abs(y[..., 0::2] - zr.real).max() < 4e-3 and np.abs(y[..., 1::2] - zr.imag).max() < 4e-3
    # position 0 is the identity
    assert (LO.rope(x[:, :1], 0, 10000.0) == x[:, :1]).all()


def test_attention_causal_gqa_against_bruteforce():
    rng = np.random.default_rng(2)
    b, s, h, hk, d, kv_len, mx = 2, 3, 4, 2, 16, 9, 12
    q = rng.standard_normal((b, s, h, d)).astype(f16)
    kc = rng.standard_normal((b, hk, mx, d)).astype(f16)
    vc = rng.standard_normal((b, hk, mx, d)).astype(f16)
    out = LO.attention(q, kc, vc, kv_len)
    for bi in range(b):
        for hi in range(h):
            for si in range(s):
                lim = kv_len - s + si + 1
                sc = np.array([np.dot(q[bi, si, hi].astype(np.float64), kc[bi, hi // 2, p].astype(np.float64)) / 4.0
                               for p in range(lim)])
                p = np.exp(sc - sc.max())
                p /= p.sum()
                want = sum(p[j] * vc[bi, hi // 2, j].astype(np.float64) for j in range(lim))
                assert np.abs(out[bi, si, hi] - want).max() < 3e-3
    # a single visible position returns that value row
    one = LO.attention(q[:, :1], kc, vc, 1)
    assert (one[0, 0, 0] == vc[0, 0, 0]).all()


def test_elementwise_and_gemv():
    rng = np.random.default_rng(3)
    g, u = rng.standard_normal(33).astype(f16), rng.standard_normal(33).astype(f16)
    want = g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64))) * u.astype(np.float64)
    assert np.abs(LO.silu_mul(g, u) - want).max() < 2e-3
    assert (LO.add(g, u) == (g.astype(np.float32) + u.astype(np.float32)).astype(f16)).all()
    w = rng.standard_normal((7, 40)).astype(f16)
    x = rng.standard_normal(40).astype(f16)
    assert np.abs(LO.fp16_gemv(w, x) - w.astype(np.float64) @ x.astype(np.float64)).max() < 2e-2
    assert (LO.fp16_gemm(x[None, :], w)[0] == LO.fp16_gemv(w, x)).all()
    t = rng.standard_normal((10, 8)).astype(f16)
    assert (LO.embedding_lookup(t, [3, 3, 9]) == t[[3, 3, 9]]).all()


def tiny_cfg(**kw):
    base = dict(vocab_size=512, hidden_dim=256, intermediate_dim=512, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=64,
                max_seq_len=64, rope_theta=10000.0, rms_norm_eps=1e-5)
    base.update(kw)
    return tf.TllmConfig(**base)


def test_forward_token_by_token_matches_one_pass():
    """Incremental decoding over the KV cache reproduces the one-pass logits (FP16 path)."""
    model = tf.random_model(tiny_cfg(), seed=5)
    toks = [5, 17, 400, 3, 99]
    a = LO.Transformer(model, int8_decode=False)
    full = a.forward(toks, 0).astype(np.float32)
    b = LO.Transformer(model, int8_decode=False)
    for i, t in enumerate(toks):
        step = b.forward([t], i)
    assert np.abs(step.astype(np.float32) - full).max() <= 2e-2 * max(1.0, np.abs(full).max())
    # the INT8 decode path stays close to the FP16 one
    c = LO.Transformer(model, int8_decode=True)
    c.forward(toks[:-1], 0)
    q = c.forward(toks[-1:], len(toks) - 1).astype(np.float32)
    assert np.abs(q - full).max() <= 0.15 * max(1.0, np.abs(full).max())
