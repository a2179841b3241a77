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


def test_mixed_layers_with_skewed_routing_run_free(cuda_device):
    """Shallow layers synchronous (their return follows the second GEMM on the side stream), deep layers displaced,
    Zipf-skewed routing, no host synchronisation between layers: the ranks drift apart and the side stream runs
    behind the main stream.  A combine wait whose dependents became resident while it spun once starved the very
    push it waited for (every rank then reported an expired wait).  The benchmark's own run of this configuration
    must finish with a clean status and a bit-identical layer 0."""
    import json

    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    root = os.path.dirname(HERE)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29633", os.path.join(root, "bench.py"), "--gpus", "2", "--shape", "g1792", "--layers", "20",
           "--steps", "3", "--warmup", "3", "--sync-steps", "1", "--ep-mode", "displaced", "--ep-async-mode", "deep",
           "--route", "zipf:1.2", "--no-full-model", "--no-gpu-reference"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=root)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-3000:])
    line = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert line["ep_parity"]["bit_identical"] and line["load"]["rows_per_rank_max_over_mean"] > 1.2
    assert line["config"]["return_of_a_sync_exchange"].startswith("follows the second GEMM")
