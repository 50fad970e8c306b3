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
    # The sharded layer-step itself: every rank holds 8 / world KV heads of one sequence's cache, runs the step
    # with the exchange inside it (LayerStepArgs.peer_gather) and must end up with the attention rows of ALL heads:
    # compared with the double-precision attention over the unsharded cache.
    if 8 % world == 0:
        from oracle import binding as orc
        from tests import helpers
        from tests.helpers import ATTN_MAX_ABS, attention_error
        from gemma_c_b200 import sharding

        orc.build()
        HQ, H, D, steps = 16, 8, 256, 3
        start = np.array([6000], np.int32)
        acase = helpers.make_append_case(77, start, window=0, ring_pages=None, max_pos=int(start[0]) + steps + 1)
        cfg_t = acase.cfg
        rng = np.random.default_rng(123)                      # the same cache on every rank
        elems = cfg_t[0] * cfg_t[1] * cfg_t[2] * cfg_t[5] * cfg_t[6]
        ck = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
        cv = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
        h_local = H // world
        my_k, my_cfg = sharding.slice_cache_heads(ck, cfg_t, world, rank)
        my_v, _ = sharding.slice_cache_heads(cv, cfg_t, world, rank)
        lo, hi = sharding.kv_head_range(H, world, rank)
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16) if a.dtype == np.uint16 else np.ascontiguousarray(a)).cuda()
        sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        ns = kv.plan_balanced(1, sms)
        hq_local = 2 * h_local
        dck, dcv = dev(my_k), dev(my_v)
        dq = torch.zeros((1, hq_local, D), dtype=torch.int16, device="cuda")
        dout = torch.zeros_like(dq)
        pm = torch.zeros(hq_local * ns, dtype=torch.float32, device="cuda")
        pl, pacc = pm.clone(), torch.zeros(hq_local * ns * D, dtype=torch.float32, device="cuda")
        ticket = torch.zeros(h_local * kv.TICKETS_PER_HEAD, dtype=torch.int32, device="cuda")
        step_buf = kv.PeerBuffer(hq_local * D * 2, world, rank)
        mine = torch.tensor(list(step_buf.export), dtype=torch.uint8, device="cuda")
        dist.all_gather_into_tensor(everyone, mine)
        step_buf.connect(bytes(everyone.cpu().tolist()))
        dist.barrier()
        table, qw, kw_, cos, sin = (dev(x) for x in (acase.page_table, acase.q_w, acase.k_w, acase.cos, acase.sin))
        qp_full = np.zeros((1, HQ, D), np.uint16)
        for t in range(steps):
            raw = [helpers.bf16_normal(rng, (1, n, D)) for n in (HQ, H, H)]       # same rows on every rank
            pos, length = (start + t).astype(np.int32), (start + t + 1).astype(np.int32)
            rq, rk, rv = dev(raw[0][:, 2 * lo:2 * hi]), dev(raw[1][:, lo:hi]), dev(raw[2][:, lo:hi])
            dpos, dlen = dev(pos), dev(length)
            a = kv.LayerStepArgs()
            a.q, a.out, a.lse = dq.data_ptr(), dout.data_ptr(), None
            a.partial_m, a.partial_l, a.partial_acc = pm.data_ptr(), pl.data_ptr(), pacc.data_ptr()
            a.cache_k, a.cache_v, a.cache_config = dck.data_ptr(), dcv.data_ptr(), kv.make_kv_config(*my_cfg)
            a.page_table, a.token_position, a.seq_lengths = table.data_ptr(), dpos.data_ptr(), dlen.data_ptr()
            a.cache_layer, a.split_size, a.num_splits, a.softmax_scale = 0, 0, ns, 1.0 / 16.0
            a.raw_q, a.raw_k, a.raw_v = rq.data_ptr(), rk.data_ptr(), rv.data_ptr()
            a.q_norm_weight, a.k_norm_weight, a.cos, a.sin = qw.data_ptr(), kw_.data_ptr(), cos.data_ptr(), sin.data_ptr()
            a.batch_count, a.q_heads, a.rotary_dim, a.norm_mode = 1, hq_local, D, kv.NORM_IEEE
            a.status, a.ticket, a.peer_gather = status.data_ptr(), ticket.data_ptr(), step_buf.handle
            assert kv.layer_step_launches(a) == 1, "the sharded step runs as the one-launch kernel"
            kv.decode_layer_step(a)
            torch.cuda.synchronize()
            assert status[0].item() == 0 and not ticket.any(), f"rank {rank} step {t}"
            got = read_device(step_buf.gathered(), world * hq_local * D // 2, np.int32).view(np.uint16)
            orc.decode_append(qp_full, ck, cv, cfg_t, acase.page_table, pos, 0, raw[0], raw[1], raw[2], acase.q_w,
                              acase.k_w, acase.cos, acase.sin, 1, HQ, D)
            ref, _ = orc.decode_attention_f64(qp_full, ck, cv, acase.page_table, length, cfg_t, 0, 1.0 / 16.0, 1, HQ)
            max_abs, _ = attention_error(got, ref)             # rank-major slots = head order
            assert max_abs <= ATTN_MAX_ABS, f"rank {rank} step {t}: gathered rows differ from the unsharded attention: {max_abs}"
        dist.barrier()
        step_buf.close()
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
