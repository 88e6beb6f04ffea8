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
