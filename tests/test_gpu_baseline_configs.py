"""Parity at the sizes BASELINE.json quotes, on the workloads bench.py times.

The other GPU tests use shapes the oracle finishes in a blink; here the CUDA path runs the bench's own workloads
(built by bench.RankWorkload from the bench's seed) at full size and a sample of its outputs is checked against
the CPU oracle with bench.verify_step -- the check the benchmark itself runs after its timed region:
  * configs[2]: 64 sequences of 512..32768 keys over a permuted pool of 16-token pages, five sliding layer-steps
    and one global one: every sequence of a sliding layer and the longest / shortest / random sequences of the
    global layer (int64 offsets into a cache of several GB, page tables of 2049 entries);
  * configs[3]: one sequence of 131072 keys with 1 % of the keys scaled x8, a table of 8193 entries, through the
    balanced partition and through fixed splits, on all 8 KV heads and on the 1-KV-head share of an 8-way shard;
  * configs[4]: 32 x 8192 keys in an FP8 e4m3 cache filled by quantise-on-append, fused-dequant decode against the
    double-precision oracle over the same quantised bytes and against the bf16 rows they were made from.
Tolerances: tests/helpers.py (attention 2^-6 abs / rel, log-sum-exp 1e-3), FP8 vs bf16 0.05 / 5e-3; appended rows:
bit-exact against the reference's own append kernel where it is built; against the IEEE host oracle no element
further than one bf16 step at its magnitude (the library's default norm mode is rsqrt.approx, like the reference's).
"""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import bench
from tests.gpu_util import dev, host_u16, host_u8, need_gpu
from tests.helpers import ATTN_MAX_ABS, ATTN_MAX_REL, LSE_MAX_ABS, attention_error

pytestmark = [pytest.mark.gpu, need_gpu]
HQ, H, D, PAGE = 16, 8, 256, 16


def _args(**kw):
    args = bench.parse_args([])
    for k, v in kw.items():
        setattr(args, k, v)
    return args


def _workload(kv, args, steps=3):
    spec, ctx_all, ctx, _, _ = bench.plan_workload(args, 1, 0)
    if args.emulate_world > 1 and args.workload in ("cfg3", "cfg5"):
        ctx = ctx_all[bench.shard_sequences(ctx_all, args.emulate_world)[args.emulate_rank]]
    wl = bench.RankWorkload(kv, torch, ctx, steps, args.seed, args, spec)
    torch.cuda.synchronize()
    return wl


def _assert_verified(res):
    assert res["ok"], res
    assert res["max_abs"] <= ATTN_MAX_ABS and res["max_rel"] <= ATTN_MAX_REL and res["lse_max_abs"] <= LSE_MAX_ABS
    a = res["append_vs_ieee_oracle"]
    assert a["beyond_one_step"] == 0 and a["differing"] <= 0.02 * max(a["elements"], 1)
    if "reference's own" in res.get("cache_checker", ""):
        assert res["cache_rows_exact"] is True


def test_config3_batch_of_the_bench(kv, orc):
    """The bench's default batch (seed 20260): two steps, then every sequence of the first sliding layer and
    eight sequences (longest, shortest, random) of the global layer."""
    args = _args(workload="cfg3")
    wl = _workload(kv, args)
    assert wl.B == 64 and int(wl.ctx.max()) > 30000 and wl.g_cfg.num_pages > 60000
    for s in range(2):
        wl.step(s)
    sliding = bench.verify_step(wl, 1, layers=[0], seqs=list(range(wl.B)))
    _assert_verified(sliding)
    assert sliding["rows"] == 64 * HQ
    glob = bench.verify_step(wl, 1, layers=[wl.timed_layer], count=8)
    _assert_verified(glob)
    order = np.argsort(wl.ctx)
    assert int(order[-1]) in glob["sequences"] and int(order[0]) in glob["sequences"]
    assert max(glob["layers"][0]["keys"]) > 30000


def test_config3_shard_of_eight_ranks(kv, orc):
    """What one of eight ranks runs (8 sequences): the small-batch form of the layer-step."""
    args = _args(workload="cfg3", emulate_world=8, emulate_rank=3)
    wl = _workload(kv, args)
    assert wl.B == 8
    for s in range(3):
        wl.step(s)
    _assert_verified(bench.verify_step(wl, 2, seqs=list(range(wl.B)), layers=[0, 2, wl.timed_layer]))


@pytest.mark.parametrize("shards", [1, 2, 8])
def test_config4_long_sequence_with_outlier_keys(kv, orc, shards):
    """131072 keys, 1 % of them x8. shards > 1: the KV heads one of `shards` ranks holds (4 or 1)."""
    args = _args(workload="cfg4", emulate_world=shards)
    wl = _workload(kv, args)
    assert wl.B == 1 and wl.g_cfg.max_pages_per_seq >= 8193 and wl.spec.hkv == 8 // shards
    for s in range(2):
        wl.step(s)
    res = bench.verify_step(wl, 1)
    _assert_verified(res)
    assert res["layers"][0]["keys"] == [131072 + 2]
    # the outliers are there: the largest key norm is several times the typical one
    rows = wl.g_k.view(-1, D)[:4096].float().norm(dim=1)
    assert rows.max().item() > 4.0 * rows.median().item()
    # the same cache through the other partition (fixed splits where the balanced one ran, and the reverse)
    i = wl.timed_layer
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    hq = wl.spec.hq
    other = []
    if wl.layers[i].split_size == 0:
        split, nsplit = kv.plan_splits_total(1, 131074, 131074, wl.spec.hkv, sms)
        other.append((split, nsplit))
    other.append((1024, -(-131074 // 1024)))
    if wl.spec.hkv == 8 and wl.layers[i].split_size != 0:
        other.append((0, kv.plan_balanced(1, sms)))
    c = bench.compact_layer_cache(wl, i, [0])
    q = bench._bits(wl.q_prepared[i])
    ref, ref_lse = orc.decode_attention_f64(q, bench._bits(c["ck"]).reshape(-1), bench._bits(c["cv"]).reshape(-1),
                                            c["table"].cpu().numpy(), wl.len_all[1].cpu().numpy(), c["cfg"], 0,
                                            1.0 / math.sqrt(D), 1, hq)
    for split, nsplit in other:
        out = torch.zeros((1, hq, D), dtype=torch.int16, device="cuda")
        lse = torch.zeros((1, hq), dtype=torch.float32, device="cuda")
        pm = torch.full((hq * nsplit,), float("nan"), dtype=torch.float32, device="cuda")
        pl, pacc = pm.clone(), torch.full((hq * nsplit * D,), float("nan"), dtype=torch.float32, device="cuda")
        st = torch.zeros(4, dtype=torch.int32, device="cuda")
        kv.decode_attention(out, lse, wl.q_prepared[i], wl.g_k, wl.g_v, wl.g_cfg, wl.g_table, wl.len_all[1], 0,
                            1.0 / math.sqrt(D), split, nsplit, 1, hq, pm, pl, pacc, st)
        torch.cuda.synchronize()
        assert st[0].item() == 0
        max_abs, max_rel = attention_error(host_u16(out), ref)
        assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (split, max_abs, max_rel)
        assert np.abs(lse.cpu().numpy() - ref_lse).max() <= LSE_MAX_ABS, split


def test_config5_fp8_batch(kv, orc):
    """32 sequences of 8192 keys in the FP8 cache. Every sequence's prompt rows come from a seed of its own, so the
    four checked ones can be replayed on the host: bytes and scales of their pages bit-exact against the oracle's
    statement of the quantisation rule (prompt fill + one decode append), attention over those bytes within the
    bf16 band of double precision, and within 0.05 / 5e-3 of the attention over the bf16 rows themselves."""
    B, ctx, seed = 32, 8192, 20260
    rng = np.random.default_rng(seed)
    pages_b = (ctx + 1 + PAGE) // PAGE
    num_pages = B * pages_b
    table = rng.permutation(num_pages).astype(np.int32).reshape(B, pages_b)
    cfg_t = (1, num_pages, PAGE, pages_b, B, H, D, 0)
    cfg = kv.make_kv_config(*cfg_t)
    elems = num_pages * PAGE * H * D
    ck = torch.zeros(elems, dtype=torch.uint8, device="cuda")
    cv = torch.zeros_like(ck)
    sk = torch.zeros(num_pages * H, dtype=torch.float32, device="cuda")
    sv = torch.zeros_like(sk)
    dtable = dev(table)

    def prompt_rows(b):
        g = torch.Generator(device="cuda")
        g.manual_seed(seed + 17 * b)
        k = torch.empty(ctx * H * D, dtype=torch.bfloat16, device="cuda").normal_(generator=g)
        v = torch.empty(ctx * H * D, dtype=torch.bfloat16, device="cuda").normal_(generator=g)
        return k, v

    one = lambda x: torch.tensor([x], dtype=torch.int32, device="cuda")
    for b in range(B):
        k, v = prompt_rows(b)
        kv.fp8_append_rows(ck, cv, sk, sv, cfg, dtable, one(b), one(0), one(ctx), one(0), 1, ctx, 0, k, v)
    raw = {n: torch.empty((B, h, D), dtype=torch.bfloat16, device="cuda").normal_() for n, h in
           (("q", HQ), ("k", H), ("v", H))}
    ones = torch.ones(D, dtype=torch.bfloat16, device="cuda")
    cos_h, sin_h = kv.fill_rope_tables(ctx + 2, D // 2, 1.0e6, D)
    cos, sin = dev(cos_h), dev(sin_h)
    pos = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    length = pos + 1
    qp = torch.zeros((B, HQ, D), dtype=torch.int16, device="cuda")
    out = torch.zeros_like(qp)
    lse = torch.zeros((B, HQ), dtype=torch.float32, device="cuda")
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    ns = kv.plan_balanced(B, sms)
    pm = torch.zeros(B * HQ * ns, dtype=torch.float32, device="cuda")
    pl, pacc = pm.clone(), torch.zeros(B * HQ * ns * D, dtype=torch.float32, device="cuda")
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(D)
    kv.decode_append_fp8(qp, ck, cv, sk, sv, cfg, dtable, pos, 0, raw["q"], raw["k"], raw["v"], ones, ones, cos, sin,
                         B, HQ, D, kv.NORM_IEEE)
    kv.decode_attention_fp8(out, lse, qp, ck, cv, sk, sv, cfg, dtable, length, 0, scale, ns, B, HQ, pm, pl, pacc, st)
    torch.cuda.synchronize()
    assert st[0].item() == 0

    picks = [0, 31, 7, 20]
    page_elems = PAGE * H * D
    w1 = orc.f32_to_bf16(np.ones(D, np.float32))
    for b in picks:
        # host replay of this sequence alone, in a cache of its own pages
        small = (1, pages_b, PAGE, pages_b, 1, H, D, 0)
        stable = np.arange(pages_b, dtype=np.int32)[None, :]
        hk, hv = np.zeros(pages_b * page_elems, np.uint8), np.zeros(pages_b * page_elems, np.uint8)
        hsk, hsv = np.zeros(pages_b * H, np.float32), np.zeros(pages_b * H, np.float32)
        k, v = prompt_rows(b)
        k_bits, v_bits = host_u16(k).reshape(ctx, H, D), host_u16(v).reshape(ctx, H, D)
        z, i32 = np.array([0], np.int32), lambda x: np.array([x], np.int32)
        orc.fp8_append(hk, hv, hsk, hsv, small, stable, z, z, i32(ctx), 0, k_bits, v_bits)
        rq, rk, rv = (host_u16(raw[n][b]).reshape(1, h, D) for n, h in (("q", HQ), ("k", H), ("v", H)))
        hq, kp, vp = orc.prefill_prep(rq, rk, rv, w1, w1, cos_h, sin_h, i32(ctx), HQ, H, D, D)
        orc.fp8_append(hk, hv, hsk, hsv, small, stable, z, i32(ctx), i32(1), 0, kp, vp)
        phys = torch.from_numpy(table[b]).long().cuda()
        got_k = host_u8(ck.view(num_pages, page_elems)[phys])
        got_v = host_u8(cv.view(num_pages, page_elems)[phys])
        assert np.array_equal(got_k, hk) and np.array_equal(got_v, hv), b
        assert np.array_equal(sk.view(num_pages, H)[phys].cpu().numpy().reshape(-1), hsk)
        assert np.array_equal(sv.view(num_pages, H)[phys].cpu().numpy().reshape(-1), hsv)
        assert np.array_equal(host_u16(qp[b]), hq.reshape(-1))
        got = host_u16(out[b]).reshape(1, HQ, D)
        ref8, lse8 = orc.fp8_decode_attention_f64(hq, hk, hv, hsk, hsv, stable, i32(ctx + 1), small, 0, scale, 1, HQ)
        max_abs, max_rel = attention_error(got, ref8)
        assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (b, max_abs, max_rel)
        assert np.abs(lse[b].cpu().numpy() - lse8.reshape(-1)).max() <= LSE_MAX_ABS
        # against the bf16 rows the cache was quantised from
        bk = np.concatenate([k_bits.reshape(-1), kp.reshape(-1), np.zeros((pages_b * PAGE - ctx - 1) * H * D, np.uint16)])
        bv = np.concatenate([v_bits.reshape(-1), vp.reshape(-1), np.zeros((pages_b * PAGE - ctx - 1) * H * D, np.uint16)])
        ref16, _ = orc.decode_attention_f64(hq, bk, bv, stable, i32(ctx + 1), small, 0, scale, 1, HQ)
        diff = np.abs(orc.bf16_to_f32(got).astype(np.float64) - ref16)
        assert diff.max() <= 0.05 and diff.mean() <= 5.0e-3, (b, diff.max(), diff.mean())


def test_config5_through_the_bench_workload(kv, orc):
    """The bench's own cfg5 workload (32 x 8192, FP8) for one step, checked the way the bench checks it."""
    wl = _workload(kv, _args(workload="cfg5"))
    wl.step(0)
    res = bench.verify_step(wl, 0, count=4)
    assert res["ok"] and res["max_abs"] <= ATTN_MAX_ABS and res["lse_max_abs"] <= LSE_MAX_ABS, res
    assert res["layers"][0]["keys"] == [8193] * 4
