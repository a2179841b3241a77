"""Expert parallelism over NCCL on 2+ GPUs of one box (skipped with fewer)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("layout", ["regions", "packed", "regions-following", "packed-following"])
def test_ep_block_over_nccl(cuda_device, layout):
    """The worker compares the block over NCCL, over peer memory (in the given receive-buffer layout: fixed regions
    per source without a count exchange, or packed blocks behind a count exchange; "-following": the return push of a
    synchronous exchange runs beside the expert FFN and follows its second GEMM) and on a single device."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 8 if n >= 8 else (4 if n >= 4 else 2)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", DICE_EP_P2P_REGIONS="1" if layout.startswith("regions") else "0",
               DICE_EP_P2P_RETURN_FOLLOWS="1" if layout.endswith("following") else "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", "29631", os.path.join(HERE, "ep_gpu_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "EP_GPU_WORKER_OK" in r.stdout, (r.stdout[-3000:], r.stderr[-3000:])
