"""b200kv_peer_allgather through the C-ABI: the all-gather of per-rank attention rows over peer memory.
One rank on one GPU exercises the kernel's own copy, flag and wait; with two or more GPUs a torchrun
job of one process per GPU compares it with NCCL's all-gather call by call (tests/peer_gather_worker.py)."""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.gpu_util import need_gpu, read_device

pytestmark = [pytest.mark.gpu, need_gpu]
REPO = Path(__file__).resolve().parent.parent


def test_single_rank_gather_copies_and_alternates_halves(kv):
    buf = kv.PeerBuffer(4096, 1, 0)
    buf.connect(buf.export)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    seen = []
    for it in range(6):
        src = torch.arange(it, it + 1024, dtype=torch.int32, device="cuda")
        ptr = buf.allgather(src, 4096, status=status)
        seen.append(ptr)
        got = read_device(ptr, 1024, np.int32)
        assert np.array_equal(got, src.cpu().numpy())
    assert status[0].item() == 0
    assert seen[0] != seen[1] and seen[0] == seen[2] and seen[1] == seen[3]
    buf.close()


def test_gather_argument_checks(kv):
    buf = kv.PeerBuffer(1024, 1, 0)
    src = torch.zeros(1024, dtype=torch.int32, device="cuda")
    assert buf.allgather(src, 2048, check=False) == 0       # larger than the slot: refused, no pointer
    assert buf.allgather(src, 24, check=False) == 0         # not a multiple of 16
    with pytest.raises(kv.CudaError):
        buf.allgather(src, 2048)
    buf.close()
    with pytest.raises(kv.CudaError):
        kv.PeerBuffer(1000, 1, 0)                            # slot size not a multiple of 16
    with pytest.raises(kv.CudaError):
        kv.PeerBuffer(1024, 9, 0)                            # more than 8 ranks


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs with peer access")
def test_two_or_more_ranks_against_nccl():
    world = min(torch.cuda.device_count(), 8)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29653", str(REPO / "tests" / "peer_gather_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(REPO))
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    assert f"PEER_GATHER_OK {world}" in proc.stdout
