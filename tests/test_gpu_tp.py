"""Tensor-parallel decoder on 2, 4 and 8 GPUs against the oracle (each case is skipped on a box with
fewer GPUs). One process per GPU under torch.distributed.run; NVLS off so that a rank that failed
could not leave the others bound to a multicast object."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_llama_matches_oracle(world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(29741 + world), os.path.join(ROOT, "tests", "tp_worker.py")]
    p = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=900)
    assert p.returncode == 0, p.stdout[-4000:]
    for r in range(world):
        assert f"TP_OK rank {r}" in p.stdout, p.stdout[-4000:]
