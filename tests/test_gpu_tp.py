"""Tensor-parallel decode on two GPUs: fused peer-memory all-reduce against the NCCL path (needs 2 GPUs)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_fused_allreduce_matches_nccl_on_two_gpus():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    worker = Path(__file__).with_name("tp_peer_worker.py")
    env = dict(os.environ, WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29533", NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(worker)], env=dict(env, RANK=str(rank), LOCAL_RANK=str(rank)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for rank in range(2)]
    outputs = []
    for proc in procs:
        try:
            out, _ = proc.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            proc.kill()
            out, _ = proc.communicate()
        outputs.append(out)
    codes = [proc.returncode for proc in procs]
    if codes == [3, 3]:
        pytest.skip("symmetric memory is not available on this system:\n" + outputs[0][-600:])
    assert codes == [0, 0], "\n".join(o[-1500:] for o in outputs)
