"""Worker of tests/test_gpu_tp_allreduce.py: one process per GPU (torch.distributed.run).
Row-parallel GEMV with the all-reduce fused into the kernel, against the oracle and
against GEMV + NCCL all-reduce."""
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
    torch.cuda.synchronize()
    dist.barrier()
    os._exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
