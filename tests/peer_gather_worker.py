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
    # key-range merge: every rank's rows and log-sum-exp against the double-precision merge
    rows, dim = 16, 256
    mbuf = kv.PeerBuffer((rows * (dim * 2 + 4) + 15) // 16 * 16, world, rank)
    mine = torch.tensor(list(mbuf.export), dtype=torch.uint8, device="cuda")
    dist.all_gather_into_tensor(everyone, mine)
    mbuf.connect(bytes(everyone.cpu().tolist()))
    dist.barrier()
    for it in range(10):
        gen.manual_seed(7000 + 10 * it + rank)
        out = torch.randn(rows, dim, device="cuda", generator=gen).bfloat16()
        lse = torch.randn(rows, device="cuda", generator=gen) * 4
        if it % 3 == 0 and rank == world - 1:
            lse[5] = float("-inf")                      # this rank saw no key of that row
        all_out = torch.empty(world, rows, dim, dtype=torch.bfloat16, device="cuda")
        all_lse = torch.empty(world, rows, dtype=torch.float32, device="cuda")
        dist.all_gather_into_tensor(all_out, out)
        dist.all_gather_into_tensor(all_lse, lse)
        merged, merged_lse = torch.empty_like(out), torch.empty_like(lse)
        mbuf.merge_attention(merged, merged_lse, out, lse, rows, dim, status=status)
        torch.cuda.synchronize()
        assert status[0].item() == 0
        w = torch.softmax(all_lse.double(), dim=0)                              # [world, rows]
        want = (w[:, :, None] * all_out.double()).sum(0)
        want_lse = torch.logsumexp(all_lse.double(), dim=0)
        err = (merged.double() - want).abs().max().item()
        assert err <= 2.0 ** -7 * max(1.0, want.abs().max().item()), f"rank {rank} merge {it}: {err}"
        assert (merged_lse.double() - want_lse).abs().max().item() <= 1e-4
    dist.barrier()
    # A rank misses a call (between steps, nothing of its own in flight): the others' waits run out after the
    # short limit set here, they report B200KV_STATUS_WAIT_TIMEOUT and return; every rank then resets its buffer
    # between two host barriers and the next matched call gathers correctly again.
    torch.cuda.synchronize()
    buf.set_wait_clocks(1 << 24)
    src = torch.full((256,), 7000 + rank, dtype=torch.int32, device="cuda")
    if rank != world - 1:
        buf.allgather(src, 1024, status=status)
        torch.cuda.synchronize()
        assert status[0].item() == kv.STATUS_WAIT_TIMEOUT, f"rank {rank}: expected the wait to run out"
        status.zero_()
    dist.barrier()
    buf.reset()
    dist.barrier()
    for it in range(3):
        src = torch.full((256,), 8000 + 10 * it + rank, dtype=torch.int32, device="cuda")
        ptr = buf.allgather(src, 1024, status=status)
        got = read_device(ptr, world * slot // 4, np.int32).reshape(world, slot // 4)[:, :256]
        assert status[0].item() == 0, f"rank {rank}: wait ran out after the reset"
        assert all((got[r] == 8000 + 10 * it + r).all() for r in range(world)), f"rank {rank}: rows after reset"
    dist.barrier()
    mbuf.close()
    buf.close()
    if rank == 0:
        print("PEER_GATHER_OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
