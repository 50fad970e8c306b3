"""The N > 1 paths on CPU: two gloo ranks partition the work the way bench.py does on GPUs and the pieces
put back together must equal the single-rank oracle result.

  * sequence sharding (no collective on the data path): every sequence is owned by exactly one rank, loads are
    balanced, and the union of the ranks' outputs is the full batch's output, bit for bit;
  * KV-head sharding (all-gather of head outputs): each rank attends over a cache that holds only its heads,
    the all-gathered rows equal the 8-head result bit for bit, and the fused append on the head slices writes
    the same bytes as the full append;
  * key-range sharding (exchange of rows + log-sum-exp, merge): each rank attends the full query over its pages
    of one long sequence through a page table that starts at its first page; the merged rows equal the
    attention over all keys within double-precision rounding.
The per-rank arithmetic is the CPU oracle here (no GPU in this suite); the GPU suite checks the kernels for
the same head counts (8, 4, 2, 1).
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = Path(__file__).resolve().parent.parent


def _worker(rank: int, world: int, port: int, result_dir: str):
    sys.path.insert(0, str(REPO))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from __graft_entry__ import load_package
        from oracle import binding as orc
        from tests.helpers import make_append_case, make_attn_case

        load_package()
        from gemma_c_b200 import sharding

        # ---- by sequence ----------------------------------------------------------------------------
        case = make_attn_case(900, [700, 33, 1500, 64, 0, 260, 1024], window=0)
        shards = sharding.shard_sequences(case.seq_lengths, world)
        mine = shards[rank]
        sub_table = np.ascontiguousarray(case.page_table[mine])
        sub_len = np.ascontiguousarray(case.seq_lengths[mine])
        sub_q = np.ascontiguousarray(case.q[mine])
        cfg = list(case.cfg)
        cfg[4] = len(mine)
        out, _ = orc.decode_attention_f64(sub_q, case.cache_k, case.cache_v, sub_table, sub_len, tuple(cfg), 0,
                                          case.scale, len(mine), 16)
        full = torch.zeros((case.batch, 16, 256), dtype=torch.float32)
        full[mine] = torch.from_numpy(out)
        owner = torch.zeros(case.batch, dtype=torch.int32)
        owner[mine] += 1
        dist.all_reduce(full)            # test-side assembly only: the data path has no collective
        dist.all_reduce(owner)
        loads = torch.zeros(world, dtype=torch.int64)
        loads[rank] = int(case.seq_lengths[mine].sum())
        dist.all_reduce(loads)

        # ---- by KV head -----------------------------------------------------------------------------
        hcase = make_attn_case(901, [900, 100], window=0)
        ck, hcfg = sharding.slice_cache_heads(hcase.cache_k, hcase.cfg, world, rank)
        cv, _ = sharding.slice_cache_heads(hcase.cache_v, hcase.cfg, world, rank)
        hq = sharding.slice_query_heads(hcase.q, 16, 8, world, rank)
        local_heads = 16 // world
        hout, hlse = orc.decode_attention_f64(hq, ck, cv, hcase.page_table, hcase.seq_lengths, hcfg, 0, hcase.scale,
                                              2, local_heads)
        gathered = [torch.empty((2, local_heads, 256), dtype=torch.float32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(hout))
        head_rows = torch.cat(gathered, dim=1)          # [batch, 16, 256] in head order

        acase = make_append_case(902, [40, 7], window=0, max_pos=64)
        elems = int(np.prod([acase.cfg[i] for i in (0, 1, 2, 5, 6)]))
        fk, fv = np.zeros(elems, np.uint16), np.zeros(elems, np.uint16)
        fq = np.zeros_like(acase.q)
        orc.decode_append(fq, fk, fv, acase.cfg, acase.page_table, acase.token_position, 0, acase.q, acase.k, acase.v,
                          acase.q_w, acase.k_w, acase.cos, acase.sin, 2, 16, 256)
        lo, hi = sharding.kv_head_range(8, world, rank)
        pk, pcfg = sharding.slice_cache_heads(np.zeros(elems, np.uint16), acase.cfg, world, rank)
        pv = pk.copy()
        pq = np.zeros((2, local_heads, 256), np.uint16)
        orc.decode_append(pq, pk, pv, pcfg, acase.page_table, acase.token_position, 0,
                          sharding.slice_query_heads(acase.q, 16, 8, world, rank),
                          np.ascontiguousarray(acase.k[:, lo:hi]), np.ascontiguousarray(acase.v[:, lo:hi]),
                          acase.q_w, acase.k_w, acase.cos, acase.sin, 2, local_heads, 256)
        want_k, _ = sharding.slice_cache_heads(fk, acase.cfg, world, rank)
        append_ok = (np.array_equal(pk, want_k) and
                     np.array_equal(pq, sharding.slice_query_heads(fq, 16, 8, world, rank)) and pk.any())
        flag = torch.tensor([int(append_ok)])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)

        # ---- by key range ---------------------------------------------------------------------------
        kcase = make_attn_case(903, [1500], window=0, outlier_frac=0.01)
        ktable, klen, _ = sharding.key_range_page_table(kcase.page_table, 1500, kcase.cfg[2], world, rank)
        kout, klse = orc.decode_attention_f64(kcase.q, kcase.cache_k, kcase.cache_v, ktable,
                                              np.array([klen], np.int32), kcase.cfg, 0, kcase.scale, 1, 16)
        rows_all = [torch.empty((1, 16, 256), dtype=torch.float32) for _ in range(world)]
        lse_all = [torch.empty((1, 16), dtype=torch.float32) for _ in range(world)]
        dist.all_gather(rows_all, torch.from_numpy(kout))
        dist.all_gather(lse_all, torch.from_numpy(klse))
        merged, merged_lse = sharding.merge_attention_rows(
            np.stack([t.numpy().reshape(16, 256) for t in rows_all]), np.stack([t.numpy().reshape(16) for t in lse_all]))

        if rank == 0:
            kref, kref_lse = orc.decode_attention_f64(kcase.q, kcase.cache_k, kcase.cache_v, kcase.page_table,
                                                      kcase.seq_lengths, kcase.cfg, 0, kcase.scale, 1, 16)
            key_err = float(np.abs(merged - kref.reshape(16, 256)).max())
            key_lse_err = float(np.abs(merged_lse - kref_lse.reshape(16)).max())
            ref, _ = orc.decode_attention_f64(case.q, case.cache_k, case.cache_v, case.page_table, case.seq_lengths,
                                              case.cfg, 0, case.scale, case.batch, 16)
            href, _ = orc.decode_attention_f64(hcase.q, hcase.cache_k, hcase.cache_v, hcase.page_table,
                                               hcase.seq_lengths, hcase.cfg, 0, hcase.scale, 2, 16)
            np.savez(os.path.join(result_dir, "result.npz"), owner=owner.numpy(), loads=loads.numpy(),
                     seq_equal=np.array_equal(full.numpy(), ref), head_equal=np.array_equal(head_rows.numpy(), href),
                     append_ok=int(flag.item()), key_err=key_err, key_lse_err=key_lse_err)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_gloo_ranks_reassemble_the_single_rank_result(tmp_path):
    world, port = 2, 29000 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    r = np.load(tmp_path / "result.npz")
    assert np.all(r["owner"] == 1)                      # every sequence owned exactly once
    assert r["loads"].max() <= 1.25 * r["loads"].mean() + 1500      # longest-first keeps ranks balanced
    assert bool(r["seq_equal"])
    assert bool(r["head_equal"])
    assert int(r["append_ok"]) == 1
    assert float(r["key_err"]) <= 1e-5 and float(r["key_lse_err"]) <= 1e-4     # fp32 rows, fp64 merge


def test_sharding_helpers(kv):
    from gemma_c_b200 import sharding

    rng = np.random.default_rng(0)
    ctx = rng.integers(512, 32769, size=64)
    for world in (1, 2, 4, 8):
        shards = sharding.shard_sequences(ctx, world)
        assert sorted(i for s in shards for i in s) == list(range(64))
        loads = [int(ctx[s].sum()) for s in shards]
        assert max(loads) - min(loads) <= ctx.max()
    table = np.arange(10, dtype=np.int32)[None, :] + 100
    t0, n0, f0 = sharding.key_range_page_table(table, 150, 16, 4, 0)
    t3, n3, f3 = sharding.key_range_page_table(table, 150, 16, 4, 3)
    assert (n0, f0, list(t0[0, :3]), t0[0, 3]) == (48, 0, [100, 101, 102], -1)
    assert (n3, f3, t3[0, 0], t3[0, 1]) == (6, 144, 109, -1)
    rows, lse = sharding.merge_attention_rows(np.ones((2, 3, 4)), np.array([[0.0, -np.inf, -np.inf], [0.0, 1.0, -np.inf]]))
    assert np.allclose(rows[0], 1.0) and np.allclose(rows[1], 1.0) and np.all(rows[2] == 0.0)
    assert np.isclose(lse[0], np.log(2.0)) and np.isclose(lse[1], 1.0) and np.isneginf(lse[2])
    assert sharding.kv_head_range(8, 4, 3) == (6, 8)
    with pytest.raises(ValueError):
        sharding.kv_head_range(8, 3, 0)
    cfg = (2, 3, 4, 3, 1, 8, 16, 0)
    cache = np.arange(2 * 3 * 4 * 8 * 16, dtype=np.uint16)
    part, pcfg = sharding.slice_cache_heads(cache, cfg, 4, 1)
    assert pcfg[5] == 2 and part.size == cache.size // 4
    assert part[0] == cache.reshape(2, 3, 4, 8, 16)[0, 0, 0, 2, 0]
