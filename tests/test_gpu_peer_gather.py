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


def test_single_rank_merge_is_the_identity(kv):
    """One rank: weight exp(lse - lse) = 1, so the merged rows are the rows; a row without keys (-inf) gives 0."""
    rows, dim = 16, 256
    buf = kv.PeerBuffer(rows * (dim * 2 + 4) + 12, 1, 0) if (rows * (dim * 2 + 4) + 12) % 16 == 0 else \
        kv.PeerBuffer((rows * (dim * 2 + 4) + 15) // 16 * 16, 1, 0)
    out = torch.randn(rows, dim, device="cuda").bfloat16()
    lse = torch.randn(rows, device="cuda") * 5
    lse[3] = float("-inf")
    merged = torch.full_like(out, float("nan"))
    merged_lse = torch.full_like(lse, float("nan"))
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    for _ in range(3):
        buf.merge_attention(merged, merged_lse, out, lse, rows, dim, status=status)
    torch.cuda.synchronize()
    assert status[0].item() == 0
    keep = [r for r in range(rows) if r != 3]
    assert torch.equal(merged[keep].view(torch.int16), out[keep].view(torch.int16))
    assert (merged[3] == 0).all() and merged_lse[3].item() == float("-inf")
    assert torch.equal(merged_lse[keep], lse[keep])
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


def test_wait_for_an_absent_rank_runs_out_and_the_next_call_works(kv):
    """The give-up path of the exchange, seen to run: a two-rank buffer on one GPU whose rank 1 is a local
    stand-in that nobody drives. With a short limit (2^22 SM clocks, a few milliseconds) rank 0's call waits for
    rank 1's flag, gives up, writes B200KV_STATUS_WAIT_TIMEOUT and returns normally; after the flag is posted in
    rank 1's name the next call finds it, leaves the status at 0 and has copied this rank's rows. Nothing
    faults, traps or hangs; the same context keeps working."""
    buf = kv.PeerBuffer(4096, 2, 0, loopback=True)
    buf.set_wait_clocks(1 << 22)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    src = torch.arange(1024, dtype=torch.int32, device="cuda")
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    start.record()
    buf.allgather(src, 4096, status=status)
    end.record()
    torch.cuda.synchronize()
    assert status[0].item() == kv.STATUS_WAIT_TIMEOUT
    assert start.elapsed_time(end) < 500.0                    # gave up promptly (the default limit is a second)
    status.zero_()
    buf.post(1, 1000)                                          # "rank 1" announces itself for every call to come
    for it in range(3):
        src = torch.arange(it, it + 1024, dtype=torch.int32, device="cuda")
        ptr = buf.allgather(src, 4096, status=status)
        got = read_device(ptr, 1024, np.int32)                # slot 0 of the gathered buffer = this rank's rows
        assert np.array_equal(got, src.cpu().numpy())
    assert status[0].item() == 0
    # an ordinary one-rank gather on the same device afterwards
    one = kv.PeerBuffer(4096, 1, 0)
    ptr = one.allgather(src, 4096, status=status)
    assert np.array_equal(read_device(ptr, 1024, np.int32), src.cpu().numpy()) and status[0].item() == 0
    one.close()
    buf.close()


def test_reset_returns_a_buffer_to_its_first_call(kv):
    buf = kv.PeerBuffer(1024, 1, 0)
    src = torch.arange(256, dtype=torch.int32, device="cuda")
    first = buf.allgather(src, 1024)
    buf.allgather(src, 1024)
    buf.allgather(src, 1024)
    buf.reset()
    assert buf.allgather(src, 1024) == first                  # the half the very first call used
    assert np.array_equal(read_device(first, 256, np.int32), src.cpu().numpy())
    buf.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs with peer access")
def test_two_or_more_ranks_against_nccl():
    world = min(torch.cuda.device_count(), 8)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29653", str(REPO / "tests" / "peer_gather_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(REPO))
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    assert f"PEER_GATHER_OK {world}" in proc.stdout


def test_key_range_shards_merge_to_the_unsharded_attention(kv, orc):
    """Key-range sharding on one GPU: the keys of a sequence are attended in two pieces (the second piece through
    a page table that starts at its first page, so its keys sit at local positions 0..), and the pieces' rows
    and log-sum-exp merged as b200kv_peer_merge_attention merges them equal the attention over all keys."""
    from tests import helpers
    from tests.gpu_util import dev, host_u16
    from tests.helpers import ATTN_MAX_ABS, ATTN_MAX_REL, LSE_MAX_ABS, attention_error

    HQ, D, total, cut = 16, 256, 2000, 1024
    case = helpers.make_attn_case(77, [total], window=0, outlier_frac=0.01)
    cfg = kv.make_kv_config(*case.cfg)
    mpps = case.cfg[3]
    tables = [case.page_table, np.concatenate([case.page_table[:, cut // 16:],
                                               np.full((1, cut // 16), -1, np.int32)], axis=1)]
    lengths = [cut, total - cut]
    assert tables[1].shape == (1, mpps)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    ns = kv.plan_balanced(1, sms)
    dq, dk, dv = dev(case.q), dev(case.cache_k), dev(case.cache_v)
    pm = torch.zeros(HQ * ns, dtype=torch.float32, device="cuda")
    pl, pacc = pm.clone(), torch.zeros(HQ * ns * D, dtype=torch.float32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    outs, lses = [], []
    for table, length in zip(tables, lengths):
        out = torch.zeros((1, HQ, D), dtype=torch.int16, device="cuda")
        lse = torch.zeros((1, HQ), dtype=torch.float32, device="cuda")
        kv.decode_attention(out, lse, dq, dk, dv, cfg, dev(table), dev(np.array([length], np.int32)), 0, case.scale,
                            0, ns, 1, HQ, pm, pl, pacc, status)
        torch.cuda.synchronize()
        outs.append(orc.bf16_to_f32(host_u16(out)).reshape(HQ, D).astype(np.float64))
        lses.append(lse.cpu().numpy().reshape(HQ).astype(np.float64))
    assert status[0].item() == 0
    lse_all = np.stack(lses)
    top = lse_all.max(0)
    weight = np.exp(lse_all - top)
    weight /= weight.sum(0)
    merged = (weight[:, :, None] * np.stack(outs)).sum(0)
    merged_lse = top + np.log(np.exp(lse_all - top).sum(0))
    ref, ref_lse = orc.decode_attention_f64(case.q, case.cache_k, case.cache_v, case.page_table,
                                            np.array([total], np.int32), case.cfg, 0, case.scale, 1, HQ)
    max_abs, max_rel = attention_error(orc.f32_to_bf16(merged.astype(np.float32)), ref)
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (max_abs, max_rel)
    assert np.abs(merged_lse - ref_lse.reshape(HQ)).max() <= LSE_MAX_ABS


def _layer_step_args(kv, case, acase, d, num_splits, ticket, status, peer):
    a = kv.LayerStepArgs()
    a.q, a.out, a.lse = d["q"].data_ptr(), d["out"].data_ptr(), None
    a.partial_m, a.partial_l, a.partial_acc = d["pm"].data_ptr(), d["pl"].data_ptr(), d["pacc"].data_ptr()
    a.cache_k, a.cache_v, a.cache_config = d["ck"].data_ptr(), d["cv"].data_ptr(), kv.make_kv_config(*acase.cfg)
    a.page_table, a.token_position, a.seq_lengths = d["table"].data_ptr(), d["pos"].data_ptr(), d["len"].data_ptr()
    a.cache_layer, a.split_size, a.num_splits, a.softmax_scale = 0, 0, num_splits, 1.0 / 16.0
    a.raw_q, a.raw_k, a.raw_v = d["rq"].data_ptr(), d["rk"].data_ptr(), d["rv"].data_ptr()
    a.q_norm_weight, a.k_norm_weight, a.cos, a.sin = (d["qw"].data_ptr(), d["kw"].data_ptr(), d["cos"].data_ptr(),
                                                      d["sin"].data_ptr())
    a.batch_count, a.q_heads, a.rotary_dim, a.norm_mode = acase.token_position.size, acase.q_heads, 256, kv.NORM_IEEE
    a.status, a.ticket, a.peer_gather = status.data_ptr(), ticket.data_ptr(), peer.handle
    return a


@pytest.mark.parametrize("name,start,window,heads", [
    ("one sequence, ring, 8 heads: one launch", [1500], 1024, 8),
    ("one sequence, linear, 2 heads (a sharded rank): one launch, grouped merge", [9000], 0, 2),
    ("forty sequences: balanced kernel + combine + gather kernel", list(range(100, 140)), 64, 8),
])
def test_layer_step_ends_with_the_gather(kv, orc, name, start, window, heads):
    """LayerStepArgs.peer_gather on one rank: after the step the gather buffer holds the step's attention rows,
    call after call (the halves alternate), whether the exchange ran inside the one-launch kernel or as the
    gather kernel behind a step of several launches."""
    from tests import helpers
    from tests.gpu_util import dev, host_u16

    rng = np.random.default_rng(5)
    start = np.asarray(start, np.int32)
    B, HQ, D = start.size, 2 * heads, 256
    acase = helpers.make_append_case(9, start, window=window, ring_pages=None, max_pos=int(start.max()) + 4,
                                     kv_heads=heads, q_heads=HQ)
    cfg_t = acase.cfg
    elems = cfg_t[0] * cfg_t[1] * cfg_t[2] * cfg_t[5] * cfg_t[6]
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    ns = kv.plan_balanced(B, sms)
    d = dict(ck=dev(orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))),
             cv=dev(orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))),
             q=torch.zeros((B, HQ, D), dtype=torch.int16, device="cuda"),
             out=torch.zeros((B, HQ, D), dtype=torch.int16, device="cuda"),
             pm=torch.zeros(B * HQ * ns, dtype=torch.float32, device="cuda"),
             pl=torch.zeros(B * HQ * ns, dtype=torch.float32, device="cuda"),
             pacc=torch.zeros(B * HQ * ns * D, dtype=torch.float32, device="cuda"),
             table=dev(acase.page_table), qw=dev(acase.q_w), kw=dev(acase.k_w), cos=dev(acase.cos), sin=dev(acase.sin),
             rq=dev(acase.q), rk=dev(acase.k), rv=dev(acase.v))
    ticket = torch.zeros(B * heads * kv.TICKETS_PER_HEAD, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    peer = kv.PeerBuffer(B * HQ * D * 2, 1, 0)
    seen = []
    for t in range(3):
        d["pos"], d["len"] = dev((start + t).astype(np.int32)), dev((start + t + 1).astype(np.int32))
        a = _layer_step_args(kv, None, acase, d, ns, ticket, status, peer)
        expected_launches = 1 if B == 1 else 3
        assert kv.layer_step_launches(a) == expected_launches, name
        kv.decode_layer_step(a)
        torch.cuda.synchronize()
        assert status[0].item() == 0 and not ticket.any()
        ptr = peer.gathered()
        seen.append(ptr)
        got = read_device(ptr, B * HQ * D // 2, np.int32).view(np.uint16)
        assert np.array_equal(got, host_u16(d["out"])), (name, t)
        assert host_u16(d["out"]).any()
    assert seen[0] != seen[1] and seen[0] == seen[2]
    peer.close()
