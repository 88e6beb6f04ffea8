"""Tensor-parallel sharding of the contraction, checked on CPU with two gloo ranks:
column shards concatenate and row shards sum (one all-reduce) to the unsharded
result.  Values come from the oracle; the unpacked ternary values of the shards
are compared bit for bit with slices of the full matrix."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle
from ternary_llm_b200 import tllm_format as tf


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, k, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    nz, sg, sc, x = oracle.make_case(n, k, seed=4242)
    full = oracle.ternary_matvec(nz, sg, sc, x[0], 128, np.float64)
    t_full = oracle.unpack_bitmasks(nz, sg)

    # column-parallel: contiguous row ranges of all three arrays (the loader's shard_ternary)
    r0, r1 = rank * n // world, (rank + 1) * n // world
    col = tf.shard_ternary(tf.TernaryTensor(nz, sg, sc), "q_proj", rank, world)
    assert np.array_equal(col.nonzero_masks, nz[r0:r1]) and np.array_equal(col.scales, sc[r0:r1])
    y_col = oracle.ternary_matvec(col.nonzero_masks, col.sign_masks, col.scales, x[0], 128, np.float64)
    gathered = [torch.zeros(r1 - r0, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(y_col))
    ok_col = np.array_equal(torch.cat(gathered).numpy(), full)
    ok_bits = np.array_equal(oracle.unpack_bitmasks(nz[r0:r1], sg[r0:r1]), t_full[r0:r1])

    # row-parallel: K ranges on 128-aligned boundaries, partial sums all-reduced
    k0, k1 = rank * k // world, (rank + 1) * k // world
    assert k0 % 128 == 0 and k1 % 128 == 0
    row = tf.shard_ternary(tf.TernaryTensor(nz, sg, sc), "o_proj", rank, world)
    nzs, sgs, scs = row.nonzero_masks, row.sign_masks, row.scales
    assert nzs.shape == (n, (k1 - k0) // 32) and np.array_equal(scs, sc[:, k0 // 128:k1 // 128])
    part = torch.from_numpy(oracle.ternary_matvec(np.ascontiguousarray(nzs), np.ascontiguousarray(sgs),
                                                  np.ascontiguousarray(scs), x[0, k0:k1], 128, np.float64))
    dist.all_reduce(part)
    bound = oracle.tolerance_bound(nz, sg, sc, x[0])
    ok_row = bool((np.abs(part.numpy() - full) <= 1e-6 * bound + 1e-12).all())
    ok_bits2 = np.array_equal(oracle.unpack_bitmasks(np.ascontiguousarray(nzs), np.ascontiguousarray(sgs)),
                              t_full[:, k0:k1])
    out[rank] = int(ok_col and ok_bits and ok_row and ok_bits2)
    dist.destroy_process_group()


def test_column_and_row_sharding_two_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Array("i", [0] * world)
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, 64, 1024, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert list(out) == [1] * world


def test_bench_tp_shapes_cover_the_full_matrices():
    import bench
    for tp in (2, 4, 8):
        shapes = dict((n, (r, c)) for n, r, c in bench.tp_shapes(tp))
        assert shapes["q"] == (8192 // tp, 8192) and shapes["o"] == (8192, 8192 // tp)
        assert shapes["gate"] == (28672 // tp, 8192) and shapes["down"] == (8192, 28672 // tp)
        assert shapes["k"] == (1024 // tp, 8192)
        for _, r, c in bench.tp_shapes(tp):
            assert r % 64 == 0 and c % 128 == 0


def _layer_worker(rank, world, port, out):
    """A whole decoder forward with the heads, the KV cache and the intermediate rows split
    over the ranks (attention stays local to a rank; the o and down partial products are
    all-reduced before the FP16 rounding) against the unsharded layer oracle."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import layer_oracle as LO
    cfg = tf.TllmConfig(vocab_size=256, hidden_dim=256, intermediate_dim=512, n_layers=2, n_heads=4, n_kv_heads=2,
                        head_dim=64, max_seq_len=16, rope_theta=10000.0, rms_norm_eps=1e-5)
    model = tf.random_model(cfg, seed=8)
    hq, hkv, hd = cfg.n_heads // world, cfg.n_kv_heads // world, cfg.head_dim
    kc = np.zeros((cfg.n_layers, 1, hkv, cfg.max_seq_len, hd), np.float16)
    vc = np.zeros_like(kc)

    def lin(t, x):              # FP32 result, not yet rounded
        return oracle.ternary_gemm(x, np.ascontiguousarray(t.nonzero_masks), np.ascontiguousarray(t.sign_masks),
                                   np.ascontiguousarray(t.scales))

    def summed(t, x):           # row-parallel: partial products summed over ranks, then rounded once
        part = torch.from_numpy(lin(t, x).astype(np.float32))
        dist.all_reduce(part)
        return part.numpy().astype(np.float16)

    def forward(tokens, start):
        n = len(tokens)
        res = LO.embedding_lookup(model.embedding, tokens)
        for li, L in enumerate(model.layers):
            sh = {k: tf.shard_ternary(L[k], k, rank, world) for k in L if k.endswith("_proj")}
            h, _ = LO.rmsnorm(res, L["attn_norm"], cfg.rms_norm_eps)
            q = lin(sh["q_proj"], h).astype(np.float16).reshape(1, n, hq, hd)
            k = lin(sh["k_proj"], h).astype(np.float16).reshape(1, n, hkv, hd)
            v = lin(sh["v_proj"], h).astype(np.float16).reshape(1, n, hkv, hd)
            q, k = LO.rope(q, start, cfg.rope_theta), LO.rope(k, start, cfg.rope_theta)
            LO.copy_to_kv_cache(k, v, kc[li], vc[li], start)
            a = LO.attention(q, kc[li], vc[li], start + n).reshape(n, -1)
            res = LO.add(res, summed(sh["o_proj"], a))
            h, _ = LO.rmsnorm(res, L["ffn_norm"], cfg.rms_norm_eps)
            act = LO.silu_mul(lin(sh["gate_proj"], h).astype(np.float16), lin(sh["up_proj"], h).astype(np.float16))
            res = LO.add(res, summed(sh["down_proj"], act))
        h, _ = LO.rmsnorm(res[-1:], model.final_norm, cfg.rms_norm_eps)
        return LO.fp16_gemv(model.lm_head, h[0])

    ref = LO.Transformer(model, int8_decode=False)
    toks = [3, 99, 200, 17, 5]
    ok = True
    got, want = forward(toks[:3], 0), ref.forward(toks[:3], 0)
    ok = ok and bool(np.abs(got.astype(np.float32) - want.astype(np.float32)).max() <= 1e-2 * max(1.0, np.abs(want).max()))
    for i in (3, 4):
        got, want = forward(toks[i:i + 1], i), ref.forward(toks[i:i + 1], i)
        ok = ok and bool(np.abs(got.astype(np.float32) - want.astype(np.float32)).max() <= 1e-2 * max(1.0, np.abs(want).max()))
    out[rank] = int(ok)
    dist.destroy_process_group()


def test_sharded_layer_forward_two_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Array("i", [0] * world)
    port = _free_port()
    procs = [ctx.Process(target=_layer_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0
    assert list(out) == [1] * world


def test_stack_config_shard_shapes_match_the_bench_shapes():
    import bench
    from ternary_llm_b200.tp_stack import StackConfig
    cfg = StackConfig(hidden=8192, n_heads=64, n_kv_heads=8, head_dim=128, intermediate=28672, max_seq_len=2048)
    for tp in (1, 2, 4, 8):
        assert cfg.shard_shapes(tp) == (bench.tp_shapes(tp) if tp > 1 else
                                        [("q", 8192, 8192), ("k", 1024, 8192), ("v", 1024, 8192), ("o", 8192, 8192),
                                         ("gate", 28672, 8192), ("up", 28672, 8192), ("down", 8192, 28672)])
    import pytest
    with pytest.raises(ValueError):
        cfg.shard_shapes(3)
