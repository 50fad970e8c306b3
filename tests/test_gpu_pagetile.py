"""The one-launch decode kernel (a CTA per sequence, KV head and key range; TMA tiles of one head's rows;
partials merged by the last CTA of a pair through tickets) on its own: b200kv_decode_attention_tiled_bf16 on
prepared rows against the double-precision oracle, over the shapes of tests/test_gpu_decode_attention.py --
rings that wrapped, ragged batches, page sizes 4 / 16 / 64, the caches of KV-head-sharded ranks (4, 2, 1 heads),
unmapped pages, empty sequences, outlier keys -- with few and many key ranges per sequence, poisoned scratch,
and many launches in a row on one scratch. (The fused form is covered by tests/test_gpu_fused_layer_step.py.)"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from tests.gpu_util import dev, host_u16, need_gpu
from tests.helpers import ATTN_MAX_ABS, ATTN_MAX_REL, LSE_MAX_ABS, attention_error, make_attn_case
from tests.test_gpu_decode_attention import CASES

pytestmark = [pytest.mark.gpu, need_gpu]


def _run(kv, case, num_splits, poison=float("nan"), repeat=1):
    cfg = kv.make_kv_config(*case.cfg)
    B, H, D = case.batch, case.q_heads, case.head_dim
    q, ck, cv = dev(case.q), dev(case.cache_k), dev(case.cache_v)
    table, seq = dev(case.page_table), dev(case.seq_lengths)
    rows = B * H * num_splits
    pm = torch.full((rows,), poison, dtype=torch.float32, device="cuda")
    pl, pacc = pm.clone(), torch.full((rows * D,), poison, dtype=torch.float32, device="cuda")
    ticket = torch.zeros(B * case.cfg[5] * kv.TICKETS_PER_HEAD, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    outs = []
    for _ in range(repeat):
        out = torch.full((B, H, D), 0x7FC0, dtype=torch.int16, device="cuda")
        lse = torch.full((B, H), float("nan"), dtype=torch.float32, device="cuda")
        kv.decode_attention_tiled(out, lse, q, ck, cv, cfg, table, seq, case.layer, case.scale, num_splits, B, H,
                                  pm, pl, pacc, ticket, status)
        outs.append((out, lse))
    torch.cuda.synchronize()
    assert status[0].item() == 0 and not ticket.any()
    for out, lse in outs[1:]:
        assert torch.equal(out, outs[0][0]) and torch.equal(lse.view(torch.int32), outs[0][1].view(torch.int32))
    return host_u16(outs[0][0]).reshape(B, H, D), outs[0][1].cpu().numpy()


def _check(orc, case, out, lse):
    ref, ref_lse = orc.decode_attention_f64(case.q, case.cache_k, case.cache_v, case.page_table, case.seq_lengths,
                                            case.cfg, case.layer, case.scale, case.batch, case.q_heads)
    assert not np.isnan(orc.bf16_to_f32(out)).any()
    max_abs, max_rel = attention_error(out, ref)
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (max_abs, max_rel)
    finite = np.isfinite(ref_lse)
    assert np.array_equal(np.isneginf(lse), np.isneginf(ref_lse))
    assert np.abs(lse[finite] - ref_lse[finite]).max(initial=0.0) <= LSE_MAX_ABS


@pytest.mark.parametrize("name", [n for n in CASES if n != "page1"])
@pytest.mark.parametrize("num_splits", [1, 3, 400])
def test_tiled_attention_matches_oracle(kv, orc, name, num_splits):
    """num_splits bounds the key ranges per (sequence, head): 1 = every pair written directly by its only CTA,
    3 = a few partials, 400 = as many ranges as the GPU has room for (up to 64)."""
    case = make_attn_case(2024, **CASES[name])
    out, lse = _run(kv, case, num_splits)
    _check(orc, case, out, lse)


def test_tiled_unmapped_pages_empty_rows_and_stale_scratch(kv, orc):
    case = make_attn_case(13, [100, 0, 40, 64, 700], window=0)
    case.page_table[0, 2] = -1
    case.page_table[2, 0] = case.cfg[1] + 5
    case.page_table[3, :] = -1
    for poison in (float("nan"), 1.0e30, -7.0):
        out, lse = _run(kv, case, 12, poison=poison, repeat=2)
        _check(orc, case, out, lse)
        assert not out[1].any() and not out[3].any()
        assert np.isneginf(lse[1]).all() and np.isneginf(lse[3]).all()
    empty = make_attn_case(14, [0, 0], window=0)
    out, lse = _run(kv, empty, 5)
    assert not out.any() and np.isneginf(lse).all()


@pytest.mark.parametrize("name,kw", [
    ("batch 1 ring", dict(seq_lens=[1500], window=1024)),
    ("eight sequences, ring", dict(seq_lens=[1500, 1024, 4000, 1025, 1100, 9000, 2048, 1030], window=1024)),
    ("one KV head of a long sequence", dict(seq_lens=[20000], window=0, kv_heads=1, q_heads=2)),      # 296 ranges: ten groups
    ("four KV heads of a long sequence", dict(seq_lens=[9000], window=0, kv_heads=4, q_heads=8)),     # 74 ranges: three groups
    ("eight KV heads, 40 ranges asked for", dict(seq_lens=[5000], window=0)),
])
def test_tiled_launches_back_to_back_give_the_same_bits(kv, orc, name, kw):
    """200 launches enqueued without a host synchronisation, every one free to start under its predecessor's tail,
    all on the same scratch and tickets: the same bits every time, no wait running out, tickets back at zero."""
    case = make_attn_case(11, **kw)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    out, lse = _run(kv, case, kv.plan_balanced(case.batch, sms), repeat=200)
    _check(orc, case, out, lse)


def test_tiled_rejects_what_it_is_not_built_for(kv):
    case = make_attn_case(3, [40], window=0, page_size=1)
    cfg = kv.make_kv_config(*case.cfg)
    buf = torch.zeros(16 * 4 * 256, dtype=torch.float32, device="cuda")
    ticket = torch.zeros(8 * kv.TICKETS_PER_HEAD, dtype=torch.int32, device="cuda")
    out = torch.zeros((1, 16, 256), dtype=torch.int16, device="cuda")
    args = (out, None, dev(case.q), dev(case.cache_k), dev(case.cache_v), cfg, dev(case.page_table),
            dev(case.seq_lengths), 0, case.scale, 4, 1, 16, buf, buf, buf)
    assert kv.decode_attention_tiled(*args, ticket, check=False) == kv.CUDA_ERROR_INVALID_VALUE   # page size 1
    ok = make_attn_case(4, [40], window=0)
    args = (out, None, dev(ok.q), dev(ok.cache_k), dev(ok.cache_v), kv.make_kv_config(*ok.cfg), dev(ok.page_table),
            dev(ok.seq_lengths), 0, ok.scale, 4, 1, 16, buf, buf, buf)
    assert kv.decode_attention_tiled(*args, None, check=False) == kv.CUDA_ERROR_INVALID_VALUE     # no tickets
    a = kv.LayerStepArgs()
    assert kv.decode_layer_step_tiled(a, stream=0, check=False) == kv.CUDA_ERROR_INVALID_VALUE


@pytest.mark.parametrize("window,start", [(64, [100, 7]), (0, [300])])
def test_decode_step_over_the_layers_of_one_cache(kv, orc, window, start):
    """b200kv_decode_step_bf16 over four cache layers with tickets, twelve steps in a row without a host
    synchronisation in between: from the second layer on a layer's kernel is told that nothing in flight writes
    its cache and streams all its keys under its predecessor's tail. Every layer, every step: cache rows and
    prepared q the oracle's bits (IEEE mode), attention within the tolerance."""
    from tests import helpers

    L, HQ, H, D, steps = 4, 16, 8, 256, 12
    rng = np.random.default_rng(91)
    start = np.asarray(start, np.int32)
    B = start.size
    acase = helpers.make_append_case(5, start, window=window, ring_pages=None if window == 0 else 5, layers=L,
                                     max_pos=int(start.max()) + steps + 1)
    cfg_t = acase.cfg
    cfg = kv.make_kv_config(*cfg_t)
    elems = cfg_t[0] * cfg_t[1] * cfg_t[2] * cfg_t[5] * cfg_t[6]
    ck = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
    cv = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
    dck, dcv = dev(ck), dev(cv)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    ns = kv.plan_balanced(B, sms)
    pm = torch.full((B * HQ * ns,), float("nan"), dtype=torch.float32, device="cuda")
    pl, pacc = pm.clone(), torch.full((B * HQ * ns * D,), float("nan"), dtype=torch.float32, device="cuda")
    ticket = torch.zeros(B * H * kv.TICKETS_PER_HEAD, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    table, qw, kw_, cos, sin = (dev(x) for x in (acase.page_table, acase.q_w, acase.k_w, acase.cos, acase.sin))
    raws = [[helpers.bf16_normal(rng, (B, n, D)) for n in (HQ, H, H)] for _ in range(steps * L)]
    draws = [[dev(x) for x in r] for r in raws]
    pos_all = [dev((start + t).astype(np.int32)) for t in range(steps)]
    len_all = [dev((start + t + 1).astype(np.int32)) for t in range(steps)]
    q = torch.zeros((steps, L, B, HQ, D), dtype=torch.int16, device="cuda")
    out = torch.zeros_like(q)
    lse = torch.zeros((steps, L, B, HQ), dtype=torch.float32, device="cuda")
    for t in range(steps):
        layers = (kv.LayerStepArgs * L)()
        for i in range(L):
            a = layers[i]
            a.q, a.out, a.lse = q[t, i].data_ptr(), out[t, i].data_ptr(), lse[t, i].data_ptr()
            a.partial_m, a.partial_l, a.partial_acc = pm.data_ptr(), pl.data_ptr(), pacc.data_ptr()
            a.cache_k, a.cache_v, a.cache_config = dck.data_ptr(), dcv.data_ptr(), cfg
            a.page_table, a.token_position, a.seq_lengths = table.data_ptr(), pos_all[t].data_ptr(), len_all[t].data_ptr()
            a.cache_layer, a.split_size, a.num_splits, a.softmax_scale = i, 0, ns, 1.0 / 16.0
            r = draws[t * L + i]
            a.raw_q, a.raw_k, a.raw_v = r[0].data_ptr(), r[1].data_ptr(), r[2].data_ptr()
            a.q_norm_weight, a.k_norm_weight, a.cos, a.sin = qw.data_ptr(), kw_.data_ptr(), cos.data_ptr(), sin.data_ptr()
            a.batch_count, a.q_heads, a.rotary_dim, a.norm_mode = B, HQ, D, kv.NORM_IEEE
            a.status, a.ticket = status.data_ptr(), ticket.data_ptr()
            assert kv.layer_step_launches(a) == 1
        kv.decode_step(layers, L)
    torch.cuda.synchronize()
    assert status[0].item() == 0 and not ticket.any()
    for t in range(steps):
        pos, length = (start + t).astype(np.int32), (start + t + 1).astype(np.int32)
        for i in range(L):
            qp = np.zeros((B, HQ, D), np.uint16)
            r = raws[t * L + i]
            orc.decode_append(qp, ck, cv, cfg_t, acase.page_table, pos, i, r[0], r[1], r[2], acase.q_w, acase.k_w,
                              acase.cos, acase.sin, B, HQ, D)
            assert np.array_equal(host_u16(q[t, i]), qp.reshape(-1)), (t, i)
            ref, ref_lse = orc.decode_attention_f64(qp, ck, cv, acase.page_table, length, cfg_t, i, 1.0 / 16.0, B, HQ)
            max_abs, max_rel = attention_error(host_u16(out[t, i]), ref)
            assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (t, i, max_abs, max_rel)
            assert np.abs(lse[t, i].cpu().numpy() - ref_lse).max() <= LSE_MAX_ABS
    assert np.array_equal(host_u16(dck), ck) and np.array_equal(host_u16(dcv), cv)


@pytest.mark.parametrize("name,window,ring_pages,start,order", [
    ("one layer, linear cache", 0, None, [300], "steps"),
    ("one layer, ring with slack", 64, 5, [100, 7], "steps"),
    ("one layer, tight ring", 64, 4, [130, 64], "steps"),
    ("two layers in turn", 64, 5, [100, 7], "alternate"),
])
def test_decode_step_with_consecutive_steps_of_a_layer_in_one_call(kv, orc, name, window, ring_pages, start, order):
    """b200kv_decode_step_bf16 with entries that name the same cache layer: they are consecutive decode steps, the
    library lets their launches overlap (a later step starts while earlier ones still run, streams its old keys
    and holds back the pages the unfinished steps write). Fourteen steps of one layer in one call -- on a linear
    cache, a ring with slack and a tight ring, where the newest row lands in the slot of a key that an unfinished
    predecessor still reads -- and seven steps of two layers in turn. Every entry: cache rows and prepared q the
    oracle's bits (IEEE mode), attention within the tolerance."""
    from tests import helpers

    HQ, H, D = 16, 8, 256
    L = 1 if order == "steps" else 2
    steps = 14 if order == "steps" else 7
    rng = np.random.default_rng(17)
    start = np.asarray(start, np.int32)
    B = start.size
    acase = helpers.make_append_case(5, start, window=window, ring_pages=ring_pages, layers=L,
                                     max_pos=int(start.max()) + steps + 1)
    cfg_t = acase.cfg
    cfg = kv.make_kv_config(*cfg_t)
    elems = cfg_t[0] * cfg_t[1] * cfg_t[2] * cfg_t[5] * cfg_t[6]
    ck = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
    cv = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
    dck, dcv = dev(ck), dev(cv)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    ns = kv.plan_balanced(B, sms)
    pm = torch.full((B * HQ * ns,), float("nan"), dtype=torch.float32, device="cuda")
    pl, pacc = pm.clone(), torch.full((B * HQ * ns * D,), float("nan"), dtype=torch.float32, device="cuda")
    ticket = torch.zeros(B * H * kv.TICKETS_PER_HEAD, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    table, qw, kw_, cos, sin = (dev(x) for x in (acase.page_table, acase.q_w, acase.k_w, acase.cos, acase.sin))
    entries = [(t, i) for t in range(steps) for i in range(L)]           # (step, layer), in launch order
    raws = [[helpers.bf16_normal(rng, (B, n, D)) for n in (HQ, H, H)] for _ in entries]
    draws = [[dev(x) for x in r] for r in raws]
    pos_all = [dev((start + t).astype(np.int32)) for t in range(steps)]
    len_all = [dev((start + t + 1).astype(np.int32)) for t in range(steps)]
    n = len(entries)
    q = torch.zeros((n, B, HQ, D), dtype=torch.int16, device="cuda")
    out = torch.zeros_like(q)
    lse = torch.zeros((n, B, HQ), dtype=torch.float32, device="cuda")
    layers = (kv.LayerStepArgs * n)()
    for e, (t, i) in enumerate(entries):
        a = layers[e]
        a.q, a.out, a.lse = q[e].data_ptr(), out[e].data_ptr(), lse[e].data_ptr()
        a.partial_m, a.partial_l, a.partial_acc = pm.data_ptr(), pl.data_ptr(), pacc.data_ptr()
        a.cache_k, a.cache_v, a.cache_config = dck.data_ptr(), dcv.data_ptr(), cfg
        a.page_table, a.token_position, a.seq_lengths = table.data_ptr(), pos_all[t].data_ptr(), len_all[t].data_ptr()
        a.cache_layer, a.split_size, a.num_splits, a.softmax_scale = i, 0, ns, 1.0 / 16.0
        r = draws[e]
        a.raw_q, a.raw_k, a.raw_v = r[0].data_ptr(), r[1].data_ptr(), r[2].data_ptr()
        a.q_norm_weight, a.k_norm_weight, a.cos, a.sin = qw.data_ptr(), kw_.data_ptr(), cos.data_ptr(), sin.data_ptr()
        a.batch_count, a.q_heads, a.rotary_dim, a.norm_mode = B, HQ, D, kv.NORM_IEEE
        a.status, a.ticket = status.data_ptr(), ticket.data_ptr()
        assert kv.layer_step_launches(a) == 1
    kv.decode_step(layers, n)
    torch.cuda.synchronize()
    assert status[0].item() == 0 and not ticket.any()
    for e, (t, i) in enumerate(entries):
        pos, length = (start + t).astype(np.int32), (start + t + 1).astype(np.int32)
        qp = np.zeros((B, HQ, D), np.uint16)
        r = raws[e]
        orc.decode_append(qp, ck, cv, cfg_t, acase.page_table, pos, i, r[0], r[1], r[2], acase.q_w, acase.k_w,
                          acase.cos, acase.sin, B, HQ, D)
        assert np.array_equal(host_u16(q[e]), qp.reshape(-1)), (name, t, i)
        ref, ref_lse = orc.decode_attention_f64(qp, ck, cv, acase.page_table, length, cfg_t, i, 1.0 / 16.0, B, HQ)
        max_abs, max_rel = attention_error(host_u16(out[e]), ref)
        assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (name, t, i, max_abs, max_rel)
        assert np.abs(lse[e].cpu().numpy() - ref_lse).max() <= LSE_MAX_ABS
    assert np.array_equal(host_u16(dck), ck) and np.array_equal(host_u16(dcv), cv)


@pytest.mark.parametrize("name,window,ring_pages,start,L,steps", [
    ("one layer, tight ring of 1024 (configs[0])", 1024, 64, [1024], 1, 32),
    ("one layer, linear", 0, None, [3000], 1, 32),
    ("six layers in turn", 1024, 65, [1500], 6, 6),
])
def test_runs_of_overlapping_launches_repeat_bit_for_bit(kv, orc, name, window, ring_pages, start, L, steps):
    """The same decode steps enqueued as runs (sixteen entries per b200kv_decode_step_bf16 call: launches start
    while their predecessors still run) twenty times over from the same initial cache: the same output bits and
    cache bytes every time, a clean status, tickets back at zero -- and the same cache bytes and prepared q as
    the steps enqueued one call at a time (the rows may differ in the last bit: runs cut the key ranges
    differently)."""
    import ctypes

    from tests import helpers

    HQ, H, D = 16, 8, 256
    rng = np.random.default_rng(5)
    start = np.asarray(start, np.int32)
    B = start.size
    acase = helpers.make_append_case(5, start, window=window, ring_pages=ring_pages, layers=L,
                                     max_pos=int(start.max()) + steps + 1)
    cfg_t = acase.cfg
    cfg = kv.make_kv_config(*cfg_t)
    elems = cfg_t[0] * cfg_t[1] * cfg_t[2] * cfg_t[5] * cfg_t[6]
    ck0 = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
    cv0 = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
    ns = kv.plan_balanced(B, torch.cuda.get_device_properties(0).multi_processor_count)
    table, qw, kw_, cos, sin = (dev(x) for x in (acase.page_table, acase.q_w, acase.k_w, acase.cos, acase.sin))
    entries = [(t, i) for t in range(steps) for i in range(L)]
    n = len(entries)
    draws = [[dev(helpers.bf16_normal(rng, (B, m, D))) for m in (HQ, H, H)] for _ in entries]
    pos_all = [dev((start + t).astype(np.int32)) for t in range(steps)]
    len_all = [dev((start + t + 1).astype(np.int32)) for t in range(steps)]

    def once(per_call):
        dck, dcv = dev(ck0), dev(cv0)
        pm = torch.full((B * HQ * ns,), float("nan"), dtype=torch.float32, device="cuda")
        pl, pacc = pm.clone(), torch.full((B * HQ * ns * D,), float("nan"), dtype=torch.float32, device="cuda")
        ticket = torch.zeros(B * H * kv.TICKETS_PER_HEAD, dtype=torch.int32, device="cuda")
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        q = torch.zeros((n, B, HQ, D), dtype=torch.int16, device="cuda")
        out = torch.zeros_like(q)
        lse = torch.zeros((n, B, HQ), dtype=torch.float32, device="cuda")
        layers = (kv.LayerStepArgs * n)()
        for e, (t, i) in enumerate(entries):
            a = layers[e]
            a.q, a.out, a.lse = q[e].data_ptr(), out[e].data_ptr(), lse[e].data_ptr()
            a.partial_m, a.partial_l, a.partial_acc = pm.data_ptr(), pl.data_ptr(), pacc.data_ptr()
            a.cache_k, a.cache_v, a.cache_config = dck.data_ptr(), dcv.data_ptr(), cfg
            a.page_table, a.token_position, a.seq_lengths = (table.data_ptr(), pos_all[t].data_ptr(),
                                                             len_all[t].data_ptr())
            a.cache_layer, a.split_size, a.num_splits, a.softmax_scale = i, 0, ns, 1.0 / 16.0
            r = draws[e]
            a.raw_q, a.raw_k, a.raw_v = r[0].data_ptr(), r[1].data_ptr(), r[2].data_ptr()
            a.q_norm_weight, a.k_norm_weight, a.cos, a.sin = (qw.data_ptr(), kw_.data_ptr(), cos.data_ptr(),
                                                              sin.data_ptr())
            a.batch_count, a.q_heads, a.rotary_dim, a.norm_mode = B, HQ, D, kv.NORM_RSQRT_APPROX
            a.status, a.ticket = status.data_ptr(), ticket.data_ptr()
        size = ctypes.sizeof(kv.LayerStepArgs)
        for e0 in range(0, n, per_call):
            m = min(per_call, n - e0)
            kv.decode_step((kv.LayerStepArgs * m).from_address(ctypes.addressof(layers) + e0 * size), m)
        torch.cuda.synchronize()
        assert status[0].item() == 0 and not ticket.any(), name
        return out, lse.view(torch.int32), q, dck, dcv

    single = once(1)
    first = once(16)
    assert all(torch.equal(a, b) for a, b in zip(first[2:], single[2:])), name       # q and caches
    worst = (first[0].view(torch.bfloat16).float() - single[0].view(torch.bfloat16).float()).abs().max().item()
    assert worst <= 2.0 ** -9, (name, worst)
    for _ in range(19):
        again = once(16)
        assert all(torch.equal(a, b) for a, b in zip(again, first)), name
