"""GPU parity of the layer operators (include/tllm_b200_layer.h) through the C ABI:
against the numpy restatement (oracle/layer_oracle.py) and, where oracle/_ref was built,
against the reference's own kernels compiled from its sources on the same inputs."""
import numpy as np
import pytest
import torch

import ternary_llm_b200 as tl
from oracle import cpu
from oracle import layer_oracle as LO
from ternary_llm_b200 import layer_ops as ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
f16 = np.float16


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


def ref_or_none():
    return cpu.ref() if cpu.have_ref() else None


def ulp_close(a, b, ulps=2.0, floor=1e-3):
    """FP16 results of the same arithmetic in a different summation order."""
    a, b = a.astype(np.float32), b.astype(np.float32)
    tol = ulps * np.maximum(np.abs(b), floor) * 2.0 ** -10
    return np.abs(a - b) <= tol


@pytest.mark.parametrize("batch,dim", [(1, 2048), (3, 4096), (2, 8192), (5, 100)])
@pytest.mark.parametrize("mode", ["plain", "residual", "residual_nostore"])
def test_rmsnorm(batch, dim, mode):
    rng = np.random.default_rng(batch * 131 + dim)
    x = rng.standard_normal((batch, dim)).astype(f16)
    r = rng.standard_normal((batch, dim)).astype(f16)
    w = (1 + 0.2 * rng.standard_normal(dim)).astype(f16)
    xd, rd, wd = dev(x), dev(r), dev(w)
    out = torch.zeros_like(xd)
    ro = torch.zeros_like(xd) if mode == "residual" else None
    ops.rmsnorm_forward(xd, wd, out, rd if mode != "plain" else None, ro, batch, dim, 1e-5)
    want, want_ro = LO.rmsnorm(x, w, 1e-5, r if mode != "plain" else None, store_residual=(mode == "residual"))
    assert ulp_close(host(out), want).all()
    if ro is not None:
        assert (host(ro) == want_ro).all()
    ref = ref_or_none()
    if ref is not None:
        out2 = torch.zeros_like(xd)
        ro2 = torch.zeros_like(xd) if ro is not None else None
        assert ref.ref_rmsnorm_forward(xd.data_ptr(), wd.data_ptr(), out2.data_ptr(),
                                       rd.data_ptr() if mode != "plain" else None,
                                       ro2.data_ptr() if ro2 is not None else None, batch, dim, 1e-5, None) == 0
        assert ulp_close(host(out), host(out2), ulps=3.0).all()
        if ro is not None:
            assert (host(ro) == host(ro2)).all()


@pytest.mark.parametrize("seq,start,hq,hk,hd", [(1, 0, 32, 8, 64), (1, 777, 8, 8, 128), (7, 5, 4, 2, 64), (33, 100, 2, 4, 32)])
def test_rope_and_cache_append(seq, start, hq, hk, hd):
    rng = np.random.default_rng(seq * 7 + start)
    b, mx, theta = 2, 1024, 500000.0
    q = rng.standard_normal((b, seq, hq, hd)).astype(f16)
    k = rng.standard_normal((b, seq, hk, hd)).astype(f16)
    v = rng.standard_normal((b, seq, hk, hd)).astype(f16)
    qd, kd = dev(q), dev(k)
    ops.rope_forward(qd, kd, b, seq, hq, hk, hd, start, theta)
    wq, wk = LO.rope(q, start, theta), LO.rope(k, start, theta)
    assert np.abs(host(qd).astype(np.float32) - wq.astype(np.float32)).max() <= 4e-3
    assert np.abs(host(kd).astype(np.float32) - wk.astype(np.float32)).max() <= 4e-3
    # append: exact copies of the rotated k and of v
    kc, vc = torch.zeros((b, hk, mx, hd), dtype=torch.float16, device=DEV), torch.zeros((b, hk, mx, hd), dtype=torch.float16, device=DEV)
    ops.copy_to_kv_cache(kd, dev(v), kc, vc, b, hk, hd, seq, start, mx)
    wkc, wvc = np.zeros((b, hk, mx, hd), f16), np.zeros((b, hk, mx, hd), f16)
    LO.copy_to_kv_cache(host(kd), v, wkc, wvc, start)
    assert (host(kc) == wkc).all() and (host(vc) == wvc).all()
    # the fused form gives the same q, k and caches
    q2, k2 = dev(q), dev(k)
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    ops.rope_append(q2, k2, dev(v), kc2, vc2, b, seq, hq, hk, hd, start, theta, mx)
    assert (host(q2) == host(qd)).all() and (host(k2) == host(kd)).all()
    assert (host(kc2) == host(kc)).all() and (host(vc2) == host(vc)).all()
    ref = ref_or_none()
    if ref is not None:
        q3, k3 = dev(q), dev(k)
        assert ref.ref_rope_forward(q3.data_ptr(), k3.data_ptr(), b, seq, hq, hk, hd, start, theta, None) == 0
        # the reference is built with fast-math sin/cos: agreement to its accuracy at these angles
        assert np.abs(host(q3).astype(np.float32) - host(qd).astype(np.float32)).max() <= 2e-2


def test_cache_append_drops_positions_past_the_end():
    b, hk, hd, mx = 1, 2, 64, 8
    k = torch.ones((b, 4, hk, hd), dtype=torch.float16, device=DEV)
    kc, vc = torch.zeros((b, hk, mx, hd), dtype=torch.float16, device=DEV), torch.zeros((b, hk, mx, hd), dtype=torch.float16, device=DEV)
    ops.copy_to_kv_cache(k, k, kc, vc, b, hk, hd, 4, 6, mx)
    got = host(kc)
    assert (got[:, :, 6:8] == 1).all() and (got[:, :, :6] == 0).all()


@pytest.mark.parametrize("hq,hk,hd", [(32, 8, 64), (8, 1, 128), (4, 4, 64), (16, 1, 64)])
@pytest.mark.parametrize("kv_len", [1, 5, 256, 257, 700])
def test_attention_decode(hq, hk, hd, kv_len):
    rng = np.random.default_rng(hq * 1000 + kv_len)
    b, mx = 2, 768
    q = rng.standard_normal((b, 1, hq, hd)).astype(f16)
    kc = rng.standard_normal((b, hk, mx, hd)).astype(f16)
    vc = rng.standard_normal((b, hk, mx, hd)).astype(f16)
    qd, kd, vd = dev(q), dev(kc), dev(vc)
    out = torch.zeros_like(qd)
    ops.attention_forward(qd, kd, vd, out, b, hq, hk, hd, 1, kv_len, mx)
    want = LO.attention(q, kc, vc, kv_len)
    assert np.abs(host(out).astype(np.float32) - want.astype(np.float32)).max() <= 4e-3
    ref = ref_or_none()
    if ref is not None:
        out2 = torch.zeros_like(qd)
        assert ref.ref_attention_forward(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), out2.data_ptr(), b, hq, hk, hd, 1,
                                         kv_len, mx, None) == 0
        assert np.abs(host(out).astype(np.float32) - host(out2).astype(np.float32)).max() <= 4e-3


@pytest.mark.parametrize("hq,hk,hd", [(32, 4, 128), (8, 1, 128), (32, 8, 64), (4, 4, 64)])
@pytest.mark.parametrize("pos,mx", [(0, 64), (63, 64), (64, 300), (2047, 2048), (1000, 2048)])
def test_fused_single_token_attention_entry_point(hq, hk, hd, pos, mx):
    """tllm_b200_attention_decode (rotary embedding, cache append and attention in one launch,
    64 cache positions per CTA, scratch owned by the library) against the three separate
    operators of the oracle, on the tensor-parallel shard geometries and cache lengths."""
    rng = np.random.default_rng(hq * 100 + pos)
    theta = 500000.0
    q = rng.standard_normal((1, 1, hq, hd)).astype(f16)
    k = rng.standard_normal((1, 1, hk, hd)).astype(f16)
    v = rng.standard_normal((1, 1, hk, hd)).astype(f16)
    kc = np.zeros((1, hk, mx, hd), f16)
    vc = np.zeros((1, hk, mx, hd), f16)
    kc[:, :, :pos] = rng.standard_normal((1, hk, pos, hd)).astype(f16)
    vc[:, :, :pos] = rng.standard_normal((1, hk, pos, hd)).astype(f16)
    qd, kd, vd, kcd, vcd = dev(q), dev(k), dev(v), dev(kc), dev(vc)
    out = torch.zeros_like(qd)
    for _ in range(2):          # a repeated step rewrites the same slot and gives the same output
        qd.copy_(dev(q))
        ops.attention_decode(qd, kd, vd, kcd[0], vcd[0], out, hq, hk, hd, pos, theta, mx)
    qr, kr = LO.rope(q, pos, theta), LO.rope(k, pos, theta)
    LO.copy_to_kv_cache(kr, v, kc, vc, pos)
    want = LO.attention(qr, kc, vc, pos + 1)
    assert np.abs(host(out).astype(np.float32) - want.astype(np.float32)).max() <= 6e-3
    assert np.abs(host(kcd).astype(np.float32) - kc.astype(np.float32)).max() <= 4e-3 and (host(vcd) == vc).all()
    tl.check_device_errors()


@pytest.mark.parametrize("seq,kv_len", [(2, 2), (33, 33), (16, 300)])
def test_attention_several_tokens_is_causal_softmax(seq, kv_len):
    rng = np.random.default_rng(seq)
    b, hq, hk, hd, mx = 1, 8, 2, 64, 320
    q = rng.standard_normal((b, seq, hq, hd)).astype(f16)
    kc = rng.standard_normal((b, hk, mx, hd)).astype(f16)
    vc = rng.standard_normal((b, hk, mx, hd)).astype(f16)
    out = torch.zeros((b, seq, hq, hd), dtype=torch.float16, device=DEV)
    ops.attention_forward(dev(q), dev(kc), dev(vc), out, b, hq, hk, hd, seq, kv_len, mx)
    want = LO.attention(q, kc, vc, kv_len)
    assert np.abs(host(out).astype(np.float32) - want.astype(np.float32)).max() <= 4e-3


@pytest.mark.parametrize("size", [1, 2, 33, 8192, 14336 * 3 + 1])
def test_silu_mul_and_add(size):
    rng = np.random.default_rng(size)
    g, u = (3 * rng.standard_normal(size)).astype(f16), rng.standard_normal(size).astype(f16)
    gd, ud = dev(g), dev(u)
    out = torch.zeros_like(gd)
    ops.silu_mul_forward(gd, ud, out, size)
    assert ulp_close(host(out), LO.silu_mul(g, u), ulps=1.0, floor=1e-4).all()
    out2 = torch.zeros_like(gd)
    ops.add_forward(gd, ud, out2, size)
    assert (host(out2) == LO.add(g, u)).all()
    ops.add_forward(gd, ud, gd, size)            # in place, as the engine calls it
    assert (host(gd) == LO.add(g, u)).all()
    ref = ref_or_none()
    if ref is not None:
        g2, o3 = dev(g), torch.zeros_like(ud)
        assert ref.ref_silu_mul_forward(g2.data_ptr(), ud.data_ptr(), o3.data_ptr(), size, None) == 0
        assert ulp_close(host(out), host(o3), ulps=2.0, floor=1e-3).all()


def test_embedding_lookup_exact():
    rng = np.random.default_rng(9)
    table = rng.standard_normal((1000, 2048)).astype(f16)
    idx = np.array([0, 999, 5, 5, 123], np.int32)
    out = torch.zeros((5, 2048), dtype=torch.float16, device=DEV)
    ops.embedding_lookup(dev(table), dev(idx), out, 5, 2048)
    assert (host(out) == table[idx]).all()
    t2 = rng.standard_normal((10, 100)).astype(f16)          # rows not 16-byte multiples
    out = torch.zeros((5, 100), dtype=torch.float16, device=DEV)
    ops.embedding_lookup(dev(t2), dev(np.array([1, 2, 3, 9, 0], np.int32)), out, 5, 100)
    assert (host(out) == t2[[1, 2, 3, 9, 0]]).all()


@pytest.mark.parametrize("rows,cols", [(1, 8), (1000, 2048), (4099, 4096), (77, 100)])
def test_fp16_gemv(rows, cols):
    rng = np.random.default_rng(rows)
    w = (0.02 * rng.standard_normal((rows, cols))).astype(f16)
    x = rng.standard_normal(cols).astype(f16)
    y = torch.zeros(rows, dtype=torch.float16, device=DEV)
    ops.fp16_gemv(dev(w), dev(x), y, rows, cols)
    exact = w.astype(np.float64) @ x.astype(np.float64)
    bound = 2e-3 * (np.abs(w.astype(np.float64)) @ np.abs(x.astype(np.float64))) + 1e-4
    assert (np.abs(host(y).astype(np.float64) - exact) <= bound).all()


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (5, 70, 33), (64, 128, 256), (130, 65, 100)])
def test_fp16_gemm(m, n, k):
    rng = np.random.default_rng(m * n)
    a = rng.standard_normal((m, k)).astype(f16)
    b = (0.05 * rng.standard_normal((n, k))).astype(f16)
    c = torch.zeros((m, n), dtype=torch.float16, device=DEV)
    ops.fp16_gemm(dev(a), dev(b), c, m, n, k)
    exact = a.astype(np.float64) @ b.astype(np.float64).T
    bound = 2e-3 * (np.abs(a.astype(np.float64)) @ np.abs(b.astype(np.float64)).T) + 1e-4
    assert (np.abs(host(c).astype(np.float64) - exact) <= bound).all()


def test_int8_gemv_with_device_scale_matches_host_scale_call():
    from ternary_llm_b200 import synth
    k = 4096
    ws, ys = [], []
    for i, n in enumerate((4096, 1024, 1024)):
        nz, sg, sc = synth.random_ternary_weight(n, k, seed=40 + i, device=DEV)
        ws.append(tl.PreparedWeight(nz, sg, sc, n, k, register=False))
        ys.append(torch.zeros(n, dtype=torch.float16, device=DEV))
    x = torch.randn(k, device=DEV).half()
    q = torch.zeros(k, dtype=torch.int8, device=DEV)
    scale = torch.zeros(1, dtype=torch.float32, device=DEV)
    tl.quantize_absmax_int8(x, q, scale, k)
    ops.ternary_gemv_int8_packed_multi(ws, q, scale, ys)
    for w, y in zip(ws, ys):
        y2 = torch.zeros_like(y)
        tl.ternary_gemv_int8_packed(w, q, float(scale.item()), y2)
        assert ulp_close(host(y), host(y2), ulps=1.0).all()


def test_argument_errors():
    x = torch.zeros(8, dtype=torch.float16, device=DEV)
    with pytest.raises(tl.TllmError):
        ops.attention_forward(x, x, x, x, 1, 3, 2, 64, 1, 1, 8)        # heads not a multiple of kv heads
    with pytest.raises(ValueError):
        ops.add_forward(x.cpu(), x, x, 8)
