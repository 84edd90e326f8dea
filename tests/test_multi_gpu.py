"""What needs more than one GPU: the exchange of output slices between real peers. Skipped on a one-GPU box; run as child
processes (one per GPU) through torch.distributed.run."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_exchange_of_slices_between_two_ranks():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29581", os.path.join(ROOT, "tests", "mgpu_child.py")], capture_output=True, text=True, timeout=600, env=env)
    assert "MGPU_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
