"""Row-parallel GEMV with the fused peer-memory all-reduce on 2 GPUs (skipped on a
single-GPU machine).  One process per GPU via torch.distributed.run on 127.0.0.1."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_allreduce_two_ranks():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(HERE, "_tp_worker.py")],
                       capture_output=True, text=True, timeout=280, env=env)
    assert r.returncode == 0 and "TP_ALLREDUCE_OK" in r.stdout and "TP_ALLREDUCE_LONG_ROWS_OK" in r.stdout and "TP_STACK_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
