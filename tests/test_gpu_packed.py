"""GPU tests of the prepared (packed) weight layout and the streaming tensor-core
GEMV that reads it: the repack is bit-exact and the results meet the same
tolerance as the general path."""
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


def _prep(nz, sg, sc, register=False):
    n, k = nz.shape[0], nz.shape[1] * 32
    return tl.PreparedWeight(_dev(nz), _dev(sg), _dev(sc), n, k, register=register)


@pytest.mark.parametrize("n,k", [(1, 128), (16, 128), (9, 384), (33, 640), (100, 1024), (1024, 4096), (4096, 4096)])
def test_repack_round_trip_bit_exact(n, k):
    nz, sg, sc, _ = oracle.make_case(n, k, seed=n + k)
    w = _prep(nz, sg, sc)
    assert w.packed.numel() == ((n + 15) // 16) * (k // 128) * 544
    nz2, sg2, sc2 = w.unpack()
    torch.cuda.synchronize()
    assert (nz2.cpu().numpy().view(np.uint32) == nz).all()
    assert (sg2.cpu().numpy().view(np.uint32) == sg).all()
    assert (sc2.cpu().numpy().view(np.uint16) == sc.view(np.uint16)).all()
    # and the decoded ternary values, through the oracle's unpacker
    assert (oracle.unpack_bitmasks(nz2.cpu().numpy().view(np.uint32), sg2.cpu().numpy().view(np.uint32))
            == oracle.unpack_bitmasks(nz, sg)).all()


def test_repack_refuses_stray_sign_bits():
    nz, sg, sc, _ = oracle.make_case(32, 256, seed=1, random_masks=True)
    with pytest.raises(tl.TllmError) as e:
        _prep(nz, sg, sc)
    assert e.value.status == -8
    # canonicalised words are accepted and decode to the same ternary values
    w = _prep(nz, sg & nz, sc)
    nz2, sg2, _ = w.unpack()
    assert (oracle.unpack_bitmasks(nz2.cpu().numpy().view(np.uint32), sg2.cpu().numpy().view(np.uint32))
            == oracle.unpack_bitmasks(nz, sg)).all()


def _run_packed(w, x):
    b = x.shape[0]
    y = torch.full((b, w.rows), float("nan"), dtype=torch.float16, device=DEV)
    tl.ternary_gemv_packed(w, _dev(x), y, b)
    torch.cuda.synchronize()
    return y.cpu().numpy()


@pytest.mark.parametrize("n,k", [(1, 128), (16, 128), (9, 384), (33, 640), (64, 1024), (1000, 2048),
                                 (1024, 4096), (4096, 4096), (8192, 2048), (4096, 11008),
                                 (14336, 4096), (4096, 14336)])
def test_gemv_packed_vs_oracle(n, k):
    nz, sg, sc, x = oracle.make_case(n, k, seed=3 * n + k)
    w = _prep(nz, sg, sc)
    y = _run_packed(w, x)
    y64, bound = exact_and_bound(nz, sg, sc, x)
    assert not np.isnan(y).any()
    assert_within(y, y64, bound, f"packed gemv {n}x{k}", slack=_half_ulp(y64))


def test_gemv_packed_signed_scales_and_dense_rows():
    n, k = 64, 512
    nz, sg, sc, x = oracle.make_case(n, k, seed=9, random_masks=True, signed_scales=True)
    sg &= nz
    nz[6], sg[6] = 0xFFFFFFFF, 0xFFFFFFFF       # all +1: largest positive group sums
    nz[7], sg[7] = 0xFFFFFFFF, 0                # all -1
    nz[3] = 0
    sg[3] = 0
    sc[4] = 0
    w = _prep(nz, sg, sc)
    y = _run_packed(w, x)
    y64, bound = exact_and_bound(nz, sg, sc, x)
    assert y[0, 3] == 0 and y[0, 4] == 0
    assert_within(y, y64, bound, "packed edge", slack=_half_ulp(y64))


def test_gemv_packed_wide_dynamic_range_and_zero_groups():
    n, k = 48, 1024
    nz, sg, sc, x = oracle.make_case(n, k, seed=21)
    x = x.astype(np.float32)
    x[0, 5] = 30000.0            # one huge activation in group 0
    x[0, 128:256] = 0.0          # an all-zero activation group
    x[0, 256:384] *= 1e-3        # a group of tiny activations
    x[0, 384:512] = 6e-8         # FP16 subnormals
    x = x.astype(np.float16)
    w = _prep(nz, sg, sc)
    y = _run_packed(w, x)
    y64, bound = exact_and_bound(nz, sg, sc, x)
    assert_within(y, y64, bound, "packed dynamic range", slack=_half_ulp(y64))


@pytest.mark.parametrize("batch", [1, 2, 3, 4, 7, 16])
def test_gemv_packed_batched(batch):
    n, k = 528, 1024
    nz, sg, sc, x = oracle.make_case(n, k, seed=50 + batch, batch=batch)
    w = _prep(nz, sg, sc)
    y = _run_packed(w, x)
    y64, bound = exact_and_bound(nz, sg, sc, x)
    assert_within(y, y64, bound, f"packed batched {batch}", slack=_half_ulp(y64))


@pytest.mark.parametrize("n,k", [(16, 128), (100, 512), (1024, 4096), (4096, 11008)])
def test_gemv_int8_packed_vs_oracle(n, k):
    nz, sg, sc, x = oracle.make_case(n, k, seed=n * 5 + k, signed_scales=True)
    q, s = oracle.quantize_absmax_int8(x[0])
    w = _prep(nz, sg, sc)
    y = torch.zeros(n, dtype=torch.float16, device=DEV)
    tl.ternary_gemv_int8_packed(w, _dev(q), float(s), y)
    torch.cuda.synchronize()
    xs = q.astype(np.float64) * np.float64(s)
    y64 = oracle.ternary_matvec(nz, sg, sc, xs, 128, np.float64)
    bound = oracle.tolerance_bound(nz, sg, sc, xs, 128)
    assert_within(y.cpu().numpy(), y64, bound, f"packed int8 {n}x{k}", slack=_half_ulp(y64))


def test_registered_weights_route_reference_signatures():
    n, k = 512, 2048
    nz, sg, sc, x = oracle.make_case(n, k, seed=77, batch=3)
    dnz, dsg, dsc, dx = _dev(nz), _dev(sg), _dev(sc), _dev(x)
    y_general = torch.zeros(3, n, dtype=torch.float16, device=DEV)
    tl.ternary_gemv_batched(dnz, dsg, dsc, dx, y_general, 3, n, k)
    w = tl.PreparedWeight(dnz, dsg, dsc, n, k, register=True)
    y_fast = torch.zeros(3, n, dtype=torch.float16, device=DEV)
    tl.ternary_gemv_batched(dnz, dsg, dsc, dx, y_fast, 3, n, k)       # same call, now packed
    y_direct = torch.zeros(3, n, dtype=torch.float16, device=DEV)
    tl.ternary_gemv_packed(w, dx, y_direct, 3)
    c = torch.zeros(3, n, dtype=torch.float16, device=DEV)
    tl.ternary_gemm(dx, dnz, dsg, dsc, c, 3, n, k)
    torch.cuda.synchronize()
    assert torch.equal(y_fast, y_direct) and torch.equal(c, y_direct)
    y64, bound = exact_and_bound(nz, sg, sc, x)
    assert_within(y_fast.cpu().numpy(), y64, bound, "registered", slack=_half_ulp(y64))
    assert_within(y_general.cpu().numpy(), y64, bound, "general", slack=_half_ulp(y64))
    w.release()
    y_again = torch.zeros(3, n, dtype=torch.float16, device=DEV)
    tl.ternary_gemv_batched(dnz, dsg, dsc, dx, y_again, 3, n, k)       # back on the general path
    torch.cuda.synchronize()
    assert torch.equal(y_again, y_general)


def test_gemv_packed_is_deterministic_and_reusable():
    n, k = 4096, 4096
    nz, sg, sc, x = oracle.make_case(n, k, seed=123)
    w = _prep(nz, sg, sc)
    dx = _dev(x)
    outs = []
    for _ in range(70):          # more launches than scratch tickets: arrival counters must self-reset
        y = torch.zeros(1, n, dtype=torch.float16, device=DEV)
        tl.ternary_gemv_packed(w, dx, y, 1)
        outs.append(y)
    torch.cuda.synchronize()
    for y in outs[1:]:
        assert torch.equal(y, outs[0])
    tl.check_device_errors()       # no bounded wait expired


def test_gemv_packed_linearity_at_full_size():
    """Size-independent property at a benchmark shape: W(2x) = 2 W(x) exactly
    (power-of-two scaling commutes with every rounding step short of overflow)."""
    n, k = 14336, 4096
    nz, sg, sc = tl.pack.random_ternary_weight(n, k, seed=4)
    w = _prep(nz, sg, sc)
    x = np.random.default_rng(8).standard_normal((1, k)).astype(np.float16)
    y1 = _run_packed(w, x)
    y2 = _run_packed(w, (2 * x.astype(np.float32)).astype(np.float16))
    normal = np.abs(y1.astype(np.float32)) >= 2.0 ** -13     # FP16 subnormals round on a fixed grid
    assert np.array_equal(2 * y1.astype(np.float32)[normal], y2.astype(np.float32)[normal])
    assert (np.abs(2 * y1.astype(np.float32) - y2.astype(np.float32)) <= 2.0 ** -23).all()
    # negation is exact up to the FP32 rounding of the two digit halves: at most one
    # FP16 ulp on a few elements
    yn = _run_packed(w, -x)
    d = np.abs(yn.astype(np.float32) + y1.astype(np.float32))
    assert (d <= np.abs(y1.astype(np.float32)) * 2.0 ** -10 + 1e-7).all() and (d > 0).mean() < 0.01


@pytest.mark.parametrize("shapes,k", [([4096, 1024, 1024], 4096), ([14336, 14336], 4096), ([64, 48], 512),
                                      ([2048, 512, 512, 100], 2048)])
def test_gemv_packed_multi_equals_separate_calls(shapes, k):
    """q/k/v- and gate/up-style fused launches give exactly what separate calls give."""
    rng = np.random.default_rng(sum(shapes) + k)
    x = rng.standard_normal(k).astype(np.float16)
    dx = _dev(x)
    ws, mats = [], []
    for i, n in enumerate(shapes):
        nz, sg, sc = tl.pack.random_ternary_weight(n, k, seed=100 + i)
        mats.append((nz, sg, sc))
        ws.append(_prep(nz, sg, sc))
    fused = [torch.full((n,), float("nan"), dtype=torch.float16, device=DEV) for n in shapes]
    tl.ternary_gemv_packed_multi(ws, dx, fused)
    single = [torch.zeros(n, dtype=torch.float16, device=DEV) for n in shapes]
    for w, y in zip(ws, single):
        tl.ternary_gemv_packed(w, dx, y, 1)
    torch.cuda.synchronize()
    for (nz, sg, sc), yf, ys in zip(mats, fused, single):
        # the fused launch may add the K groups in a different order: at most a last-place difference
        d = (yf.float() - ys.float()).abs()
        assert bool((d <= ys.float().abs() * 2.0 ** -10 + 1e-6).all())
        y64, bound = exact_and_bound(nz, sg, sc, x)
        assert_within(yf.cpu().numpy(), y64, bound, "fused", slack=_half_ulp(y64))


def test_tllm_file_to_prepared_weights(tmp_path):
    """Writer -> file -> loader -> kernels: every projection of a small random-init model."""
    from ternary_llm_b200 import tllm_format as tf
    cfg = tf.TllmConfig(vocab_size=64, hidden_dim=256, intermediate_dim=512, n_layers=2, n_heads=4,
                        n_kv_heads=2, head_dim=64, max_seq_len=64)
    m = tf.random_model(cfg, seed=11)
    path = str(tmp_path / "tiny.tllm")
    tf.write_tllm(path, m)
    cfg2, layers = tf.load_projections(path, DEV)
    assert cfg2 == cfg and len(layers) == 2
    rng = np.random.default_rng(5)
    for li, layer in enumerate(layers):
        for name in tf.PROJ_NAMES:
            w = layer[name]
            t = m.layers[li][name]
            x = rng.standard_normal((1, w.cols)).astype(np.float16)
            y = _run_packed(w, x)
            y64, bound = exact_and_bound(t.nonzero_masks, t.sign_masks, t.scales, x)
            assert_within(y, y64, bound, f"L{li}.{name}", slack=_half_ulp(y64))


def test_tllm_file_sharded_load(tmp_path):
    """Shard-at-load: two tensor-parallel ranks' loads of one file (verified repack, q|k|v and
    gate|up grouped) reassemble every projection -- column shards stacked, row shards summed."""
    from ternary_llm_b200 import tllm_format as tf
    cfg = tf.TllmConfig(vocab_size=64, hidden_dim=512, intermediate_dim=1024, n_layers=1, n_heads=8,
                        n_kv_heads=2, head_dim=64, max_seq_len=64)
    m = tf.random_model(cfg, seed=12)
    path = str(tmp_path / "tp.tllm")
    tf.write_tllm(path, m)
    world = 2
    ranks = [tf.load_projections(path, DEV, rank=r, world=world, verify=True, grouped=True)[1][0] for r in range(world)]
    for r in range(world):      # grouped: the packed matrices of a group lie back to back
        q, k, v = (ranks[r][n] for n in ("q_proj", "k_proj", "v_proj"))
        assert k.packed.data_ptr() == q.packed.data_ptr() + q.packed.numel()
        assert v.packed.data_ptr() == k.packed.data_ptr() + k.packed.numel()
    rng = np.random.default_rng(6)
    for name, rows, cols in cfg.proj_shapes():
        t = m.layers[0][name]
        x = rng.standard_normal((1, cols)).astype(np.float16)
        y64, bound = exact_and_bound(t.nonzero_masks, t.sign_masks, t.scales, x)
        if name in tf.TP_COLUMN:
            assert all(ranks[r][name].rows == rows // world and ranks[r][name].cols == cols for r in range(world))
            y = np.concatenate([_run_packed(ranks[r][name], x) for r in range(world)], axis=-1)
            assert_within(y, y64, bound, name, slack=_half_ulp(y64))
        else:
            kw = cols // world
            assert all(ranks[r][name].rows == rows and ranks[r][name].cols == kw for r in range(world))
            parts = [_run_packed(ranks[r][name], np.ascontiguousarray(x[:, r * kw:(r + 1) * kw])).astype(np.float64)
                     for r in range(world)]
            # each partial result is rounded to FP16 once before the sum
            assert_within(sum(parts), y64, bound, name, slack=sum(_half_ulp(p) for p in parts))
    # the fused launch over a group read through the loader's layout
    x = torch.randn(cfg.hidden_dim, device=DEV).half()
    g = [ranks[1][n] for n in ("gate_proj", "up_proj")]
    ys = [torch.zeros(w.rows, dtype=torch.float16, device=DEV) for w in g]
    tl.ternary_gemv_packed_multi(g, x, ys)
    for w, y in zip(g, ys):
        y1 = torch.zeros_like(y)
        tl.ternary_gemv_packed(w, x, y1, 1)
        torch.cuda.synchronize()
        assert (y.float() - y1.float()).abs().max().item() <= 2.0 ** -10 * max(1.0, y1.float().abs().max().item())
    with pytest.raises(ValueError):
        tf.load_projections(path, DEV, rank=0, world=16)       # 512 columns / 16 ranks is no whole group


def test_group_packed_back_to_back_runs_as_one_matrix():
    """prepare_group + the fused entry points: same results as one call per matrix, FP16 and INT8."""
    from ternary_llm_b200 import layer_ops, synth
    k = 2048
    shapes = (1024, 256, 272)          # the last row count need not be a multiple of 16
    mats = []
    for i, n in enumerate(shapes):
        nz, sg, sc = synth.random_ternary_weight(n, k, seed=70 + i, device="cuda")
        mats.append((nz, sg, sc, n, k))
    group = tl.prepare_group(mats)
    assert all(group[i + 1].packed.data_ptr() == group[i].packed.data_ptr() + group[i].packed.numel() for i in range(2))
    x = torch.randn(k, device="cuda").half()
    ys = [torch.zeros(n, dtype=torch.float16, device="cuda") for n in shapes]
    tl.ternary_gemv_packed_multi(group, x, ys)
    for w, y in zip(group, ys):
        y1 = torch.zeros_like(y)
        tl.ternary_gemv_packed(w, x, y1, 1)
        torch.cuda.synchronize()
        # the split over CTAs differs between the two launches, hence the order of the FP32 partial sums
        assert (y.float().cpu() - y1.float().cpu()).abs().max() <= 2.0 ** -10 * max(1.0, float(y1.float().abs().max()))
    q = torch.zeros(k, dtype=torch.int8, device="cuda")
    scale = torch.zeros(1, dtype=torch.float32, device="cuda")
    tl.quantize_absmax_int8(x, q, scale, k)
    yi = [torch.zeros(n, dtype=torch.float16, device="cuda") for n in shapes]
    layer_ops.ternary_gemv_int8_packed_multi(group, q, scale, yi)
    for w, y in zip(group, yi):
        y1 = torch.zeros_like(y)
        tl.ternary_gemv_int8_packed(w, q, float(scale.item()), y1)
        torch.cuda.synchronize()
        assert (y.float().cpu() - y1.float().cpu()).abs().max() <= 2.0 ** -10 * max(1.0, float(y1.float().abs().max()))
    tl.check_device_errors()
