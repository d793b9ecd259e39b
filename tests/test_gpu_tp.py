"""Tensor-parallel decode on 2, 4 and 8 GPUs: the fused peer-memory exchanges against the NCCL path."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_exchanges_match_nccl(world):
    """toy128 has 2 kv heads, so 4 and 8 ranks use the 8-kv-head variant toy128x8."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} CUDA devices")
    worker = Path(__file__).with_name("tp_peer_worker.py")
    env = dict(os.environ, WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29533 + world), NCCL_NVLS_ENABLE="0",
               TX_TP_CONFIG="toy128" if world == 2 else "toy128x8")
    procs = [subprocess.Popen([sys.executable, str(worker)], env=dict(env, RANK=str(rank), LOCAL_RANK=str(rank)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for rank in range(world)]
    outputs = []
    for proc in procs:
        try:
            out, _ = proc.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            proc.kill()
            out, _ = proc.communicate()
        outputs.append(out)
    codes = [proc.returncode for proc in procs]
    if set(codes) == {3}:
        pytest.skip("symmetric memory is not available on this system:\n" + outputs[0][-600:])
    assert codes == [0] * world, "\n".join(o[-1500:] for o in outputs)
