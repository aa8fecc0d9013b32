"""Context-parallel decode on 2 GPUs against the single-GPU hot path (needs a
box with at least two GPUs; one rank per GPU under torchrun, NCCL)."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
@pytest.mark.parametrize("transport", ["fused", "peer", "nccl"])
@pytest.mark.parametrize("seq_len", [40005, 4099])
def test_context_parallel_matches_single_gpu(seq_len, transport):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, CP_SEQ_LEN=str(seq_len), CP_TRANSPORT=transport,
               NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29631", os.path.join(HERE, "cp_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
