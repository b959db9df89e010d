"""The fused all-reduce + residual + RMSNorm kernel on real peer memory: one process per GPU (needs >= 2 GPUs;
skipped otherwise -- the single-GPU suite covers the same kernel through the emulated communicator)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run_ranks(script, world, port, marker):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world),
               NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", script)],
                              env=dict(env, RANK=str(r)), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(world)]
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=300)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append(p.communicate()[0] + "\n[timed out]")
    assert all(p.returncode == 0 for p in procs), "\n".join(o[-2000:] for o in outs)
    assert all(f"{marker} {r}" in outs[r] for r in range(world))
    return outs


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("world", [2, 4, 8])
def test_allreduce_across_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_ranks("tp_allreduce_worker.py", world, 29620 + world, "TP_ALLREDUCE_OK")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_engine_matches_single_gpu_engine(world):
    """Hidden states at the LM head, TP = world against TP = 1 on the same requests, on real GPUs."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    outs = _run_ranks("tp_engine_worker.py", world, 29640 + world, "TP_ENGINE_OK")
    print(outs[0][-200:])
