"""Peer-memory decode across real GPUs: needs at least two devices in one box (skipped
otherwise).  Ranks are child processes; NVLS is switched off in NCCL and the symmetric memory
is asked not to bind multicast, the decode itself uses plain peer loads only."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one box")
def test_two_ranks_decode_from_each_others_memory():
    world = 2
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29541", WORLD_SIZE=str(world),
               NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    procs = []
    for rank in range(world):
        procs.append(subprocess.Popen(
            [sys.executable, os.path.join(ROOT, "tests", "peer_worker.py")],
            env=dict(env, RANK=str(rank), LOCAL_RANK=str(rank)),
            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outputs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outputs.append(out)
    for rank, (p, out) in enumerate(zip(procs, outputs)):
        assert p.returncode == 0 and f"PEER-OK rank {rank}" in out, out[-2000:]
