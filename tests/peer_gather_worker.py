"""Worker of tests/test_gpu_peer_gather.py: one process per GPU (torchrun), the peer-memory all-gather
against NCCL's on the same data, many calls in a row, sizes up to the slot. Prints PEER_GATHER_OK on rank 0."""
from __future__ import annotations

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from tests.conftest import load_package  # noqa: E402
from tests.gpu_util import read_device  # noqa: E402

import numpy as np  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    kv = load_package()
    kv.load_library(build_if_missing=False)
    slot = 8192
    buf = kv.PeerBuffer(slot, world, rank)
    mine = torch.tensor(list(buf.export), dtype=torch.uint8, device="cuda")
    everyone = torch.empty(world * 64, dtype=torch.uint8, device="cuda")
    dist.all_gather_into_tensor(everyone, mine)
    buf.connect(bytes(everyone.cpu().tolist()))
    dist.barrier()
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    gen = torch.Generator(device="cuda")
    for it in range(60):
        words = [2048, 4, 512, 1024][it % 4]           # int32 words: 16 B .. the whole slot
        gen.manual_seed(1000 * it + rank)
        src = torch.randint(-2 ** 31, 2 ** 31 - 1, (words,), dtype=torch.int32, device="cuda", generator=gen)
        want = torch.empty(world * words, dtype=torch.int32, device="cuda")
        dist.all_gather_into_tensor(want, src)
        ptr = buf.allgather(src, words * 4, status=status)
        got = read_device(ptr, world * slot // 4, np.int32).reshape(world, slot // 4)[:, :words].reshape(-1)
        assert status[0].item() == 0, f"rank {rank} call {it}: a wait ran out"
        assert np.array_equal(got, want.cpu().numpy()), f"rank {rank} call {it}: gathered rows differ"
    # back to back without reading in between: ranks run ahead of one another by at most one call
    srcs = [torch.full((256,), 100 * i + rank, dtype=torch.int32, device="cuda") for i in range(40)]
    ptrs = [buf.allgather(s, 1024, status=status) for s in srcs]
    got = read_device(ptrs[-1], world * slot // 4, np.int32).reshape(world, slot // 4)[:, :256]
    assert status[0].item() == 0
    assert all((got[r] == 100 * 39 + r).all() for r in range(world))
    dist.barrier()
    buf.close()
    if rank == 0:
        print("PEER_GATHER_OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
