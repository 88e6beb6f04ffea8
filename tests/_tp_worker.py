"""Worker of tests/test_gpu_tp_allreduce.py: one process per GPU (torch.distributed.run).
Row-parallel GEMV with the all-reduce fused into the kernel, against the oracle and
against GEMV + NCCL all-reduce; then the tensor-parallel layer stack (attention included)
against the unsharded layer oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import ternary_llm_b200 as tl  # noqa: E402
from oracle import oracle  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    n, k = 4096, 1024 * world
    nz, sg, sc, x = oracle.make_case(n, k, seed=77)          # same on every rank
    k0, k1 = rank * k // world, (rank + 1) * k // world
    nzs = np.ascontiguousarray(nz[:, k0 // 32:k1 // 32])
    sgs = np.ascontiguousarray(sg[:, k0 // 32:k1 // 32])
    scs = np.ascontiguousarray(sc[:, k0 // 128:k1 // 128])

    def d(a):
        return torch.from_numpy(a.view(np.int32) if a.dtype == np.uint32 else a).to(dev)

    w = tl.PreparedWeight(d(nzs), d(sgs), d(scs), n, k1 - k0, register=False)
    xs = d(np.ascontiguousarray(x[0, k0:k1]))
    ar = tl.FusedAllReduce(dist.group.WORLD, n, dev)
    ok = True
    outs = []
    for rep in range(5):                                       # odd and even buffer parities, reuse
        y = torch.full((n,), float("nan"), dtype=torch.float16, device=dev)
        tl.ternary_gemv_packed_allreduce(w, xs, y, ar)
        outs.append(y)
    torch.cuda.synchronize()
    tl.check_device_errors()
    y_nccl = torch.zeros(n, dtype=torch.float16, device=dev)
    tl.ternary_gemv_packed(w, xs, y_nccl, 1)
    y32 = y_nccl.float()
    dist.all_reduce(y32)
    torch.cuda.synchronize()
    y64 = oracle.ternary_matvec(nz, sg, sc, x[0], 128, np.float64)
    bound = oracle.tolerance_bound(nz, sg, sc, x[0])
    half_ulp = 0.5 * 2.0 ** (np.floor(np.log2(np.maximum(np.abs(y64), 2.0 ** -14))) - 10)
    for y in outs:
        ok = ok and bool(torch.equal(y, outs[0]))
        err = np.abs(y.cpu().numpy().astype(np.float64) - y64)
        ok = ok and bool((err <= bound + half_ulp).all())
    # all ranks hold the same result
    gathered = [torch.zeros_like(outs[0]) for _ in range(world)]
    dist.all_gather(gathered, outs[0])
    ok = ok and all(bool(torch.equal(g, gathered[0])) for g in gathered)
    # and it agrees with the NCCL route up to FP16 rounding of the per-rank partial sums
    ok = ok and bool(((outs[0].float() - y32).abs() <= y32.abs() * 2.0 ** -8 + 2e-2).all())
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("TP_ALLREDUCE_OK" if int(flag.item()) == 1 else "TP_ALLREDUCE_FAIL", flush=True)

    # long rows: the launch runs as clusters of two CTAs that split this rank's columns, and the
    # first CTA of each cluster takes part in the exchange between the ranks
    n2, k2 = 4096, 14336 * world
    nz2, sg2, sc2, x2 = oracle.make_case(n2, k2, seed=78)
    c0, c1 = rank * k2 // world, (rank + 1) * k2 // world
    w2 = tl.PreparedWeight(d(np.ascontiguousarray(nz2[:, c0 // 32:c1 // 32])), d(np.ascontiguousarray(sg2[:, c0 // 32:c1 // 32])),
                           d(np.ascontiguousarray(sc2[:, c0 // 128:c1 // 128])), n2, c1 - c0, register=False)
    xs2 = d(np.ascontiguousarray(x2[0, c0:c1]))
    outs2 = []
    for rep in range(3):
        y = torch.full((n2,), float("nan"), dtype=torch.float16, device=dev)
        tl.ternary_gemv_packed_allreduce(w2, xs2, y, ar)
        outs2.append(y)
    torch.cuda.synchronize()
    tl.check_device_errors()
    rows2 = np.unique(np.concatenate([np.arange(64), np.arange(n2 - 64, n2), np.random.default_rng(3).integers(0, n2, 256)]))
    y64b = oracle.ternary_matvec(nz2[rows2], sg2[rows2], sc2[rows2], x2[0], 128, np.float64)
    boundb = oracle.tolerance_bound(nz2[rows2], sg2[rows2], sc2[rows2], x2[0])
    half_ulp_b = 0.5 * 2.0 ** (np.floor(np.log2(np.maximum(np.abs(y64b), 2.0 ** -14))) - 10)
    ok3 = all(bool(torch.equal(y, outs2[0])) for y in outs2)
    ok3 = ok3 and bool((np.abs(outs2[0].cpu().numpy().astype(np.float64)[rows2] - y64b) <= boundb + half_ulp_b).all())
    flag3 = torch.tensor([1 if ok3 else 0], device=dev)
    dist.all_reduce(flag3, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("TP_ALLREDUCE_LONG_ROWS_OK" if int(flag3.item()) == 1 else "TP_ALLREDUCE_LONG_ROWS_FAIL", flush=True)
    flag = torch.minimum(flag, flag3)

    # the whole layer stack, heads and intermediate rows split over the ranks, fused exchange:
    # logits from the replicated residual stream against the unsharded layer oracle
    from oracle import layer_oracle as LO
    from ternary_llm_b200 import tllm_format as tf
    from ternary_llm_b200.tp_stack import StackConfig, TpLayerStack, layer_sources_from_model
    cfg = tf.TllmConfig(vocab_size=512, hidden_dim=1024, intermediate_dim=2048, n_layers=2, n_heads=8, n_kv_heads=world,
                        head_dim=128, max_seq_len=32, rope_theta=10000.0, rms_norm_eps=1e-5)
    model = tf.random_model(cfg, seed=31)                      # the same on every rank
    sc_ = StackConfig(hidden=cfg.hidden_dim, n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                      intermediate=cfg.intermediate_dim, max_seq_len=cfg.max_seq_len, rope_theta=cfg.rope_theta,
                      rms_norm_eps=cfg.rms_norm_eps)
    stack = TpLayerStack(sc_, layer_sources_from_model(model, rank, world, dev), rank, world, dev, dist.group.WORLD,
                         allreduce="fused", batch=1)
    emb = torch.from_numpy(model.embedding).to(dev)
    ref = LO.Transformer(model, int8_decode=False)
    ok2 = True
    for pos, tok in enumerate([7, 300, 41, 5]):
        res = stack.step(emb[tok:tok + 1].contiguous(), pos).float().cpu().numpy()
        want = ref.forward([tok], pos).astype(np.float32)
        h, _ = LO.rmsnorm(res.astype(np.float16), model.final_norm, cfg.rms_norm_eps)
        got = LO.fp16_gemv(model.lm_head, h[0]).astype(np.float32)
        ok2 = ok2 and bool(np.isfinite(res).all()) and bool(np.abs(got - want).max() <= 4e-2 * max(1.0, np.abs(want).max()))
    tl.check_device_errors()
    flag2 = torch.tensor([1 if ok2 else 0], device=dev)
    dist.all_reduce(flag2, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("TP_STACK_OK" if int(flag2.item()) == 1 else "TP_STACK_FAIL", flush=True)
    flag = torch.minimum(flag, flag2)
    torch.cuda.synchronize()
    dist.barrier()
    os._exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
