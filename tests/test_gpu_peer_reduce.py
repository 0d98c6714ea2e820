"""The data-parallel gradient exchange with its reduce half inside the weight-gradient GEMMs (adds into the owner
rank's memory over NVLink) against NCCL's all-reduce: needs two GPUs, skipped on a single-GPU machine."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
def test_peer_reduce_equals_nccl_allreduce_on_two_ranks():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29517", os.path.join(HERE, "peer_reduce_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0 and "PEER_REDUCE_OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]
