"""GPU parity of the split-KV flash-decode + combine, through the C-ABI, against the
double-precision CPU oracle on the same bf16 cache.

Stated tolerance (bf16 outputs): max_abs <= 2^-6 and max_rel <= 2^-6 with the denominator
max(|a|, |b|, 1); log-sum-exp: |delta| <= 1e-3. Edge cases follow the reference source:
empty rows give zeros, over-provisioned splits leave the scratch untouched, unmapped pages
contribute nothing, splits start at first_key and may straddle pages.
"""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from tests.gpu_util import dev, host_u16, need_gpu
from tests.helpers import ATTN_MAX_ABS, ATTN_MAX_REL, LSE_MAX_ABS, attention_error, make_attn_case

pytestmark = [pytest.mark.gpu, need_gpu]


class DeviceCase:
    def __init__(self, kv, case):
        self.kv, self.case = kv, case
        self.cfg = kv.make_kv_config(*case.cfg)
        self.q, self.ck, self.cv = dev(case.q), dev(case.cache_k), dev(case.cache_v)
        self.table, self.seq = dev(case.page_table), dev(case.seq_lengths)

    def run(self, split_size, num_splits, poison=None, want_lse=True):
        c, kv = self.case, self.kv
        B, H, D = c.batch, c.q_heads, c.head_dim
        out = torch.full((B, H, D), 0x7FC0, dtype=torch.int16, device="cuda")     # bf16 NaN pattern
        lse = torch.full((B, H), float("nan"), dtype=torch.float32, device="cuda") if want_lse else None
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        pm = pl = pacc = None
        if num_splits > 1:
            fill = float("nan") if poison is None else poison
            pm = torch.full((B * H * num_splits,), fill, dtype=torch.float32, device="cuda")
            pl = torch.full_like(pm, fill)
            pacc = torch.full((B * H * num_splits * D,), fill, dtype=torch.float32, device="cuda")
        kv.decode_attention(out, lse, self.q, self.ck, self.cv, self.cfg, self.table, self.seq, c.layer, c.scale,
                            split_size, num_splits, B, H, pm, pl, pacc, status)
        torch.cuda.synchronize()
        assert status[0].item() == kv.STATUS_OK
        return (host_u16(out).reshape(B, H, D), None if lse is None else lse.cpu().numpy(),
                None if pm is None else pm.cpu().numpy().reshape(B, H, num_splits))


def check(orc, case, out, lse):
    ref, ref_lse = orc.decode_attention_f64(case.q, case.cache_k, case.cache_v, case.page_table, case.seq_lengths,
                                            case.cfg, case.layer, case.scale, case.batch, case.q_heads)
    assert not np.isnan(orc.bf16_to_f32(out)).any()
    max_abs, max_rel = attention_error(out, ref)
    assert max_abs <= ATTN_MAX_ABS, max_abs
    assert max_rel <= ATTN_MAX_REL, max_rel
    if lse is not None:
        finite = np.isfinite(ref_lse)
        assert np.array_equal(np.isneginf(lse), np.isneginf(ref_lse))
        assert np.abs(lse[finite] - ref_lse[finite]).max(initial=0.0) <= LSE_MAX_ABS
    return max_abs


def live_keys(case):
    w = case.cfg[7]
    return [min(int(s), w) if w > 0 else int(s) for s in case.seq_lengths]


CASES = {
    "config1_tight_ring_wrapped": dict(seq_lens=[1025], window=1024, ring_pages=64),
    "slack_ring_wrapped": dict(seq_lens=[1041], window=1024),
    "ring_not_yet_full": dict(seq_lens=[700], window=1024),
    "linear_4096": dict(seq_lens=[4096], window=0),
    "mixed_batch": dict(seq_lens=[300, 17, 1, 64, 129, 2047, 8], window=0),
    "mixed_batch_ring": dict(seq_lens=[5000, 90, 1024, 1023, 1025], window=1024),
    "page64": dict(seq_lens=[1000, 65], window=0, page_size=64),
    "page4": dict(seq_lens=[77, 31], window=0, page_size=4),
    "page8": dict(seq_lens=[333, 50], window=0, page_size=8),
    "page1": dict(seq_lens=[40], window=0, page_size=1),
    "outliers": dict(seq_lens=[3000], window=0, outlier_frac=0.01),
    "layer1_of_3": dict(seq_lens=[500, 33], window=0, layers=3, layer=1),
    "kv4_shard": dict(seq_lens=[900, 100], window=0, kv_heads=4, q_heads=8),
    "kv2_shard": dict(seq_lens=[900, 100], window=0, kv_heads=2, q_heads=4),
    "kv1_shard": dict(seq_lens=[900, 100], window=0, kv_heads=1, q_heads=2),
}


@pytest.mark.parametrize("name", list(CASES))
@pytest.mark.parametrize("split", ["one", "tile", "ref20", "ragged_overprovisioned", "balanced"])
def test_decode_attention_matches_oracle(kv, orc, name, split):
    case = make_attn_case(2024, **CASES[name])
    longest = max(live_keys(case))
    if split == "balanced":
        if case.kv_heads != 8:
            pytest.skip("balanced partition is built for 8 KV heads")
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        split_size, num_splits = 0, kv.plan_balanced(case.batch, sms)
    elif split == "one":
        split_size, num_splits = max(longest, 1), 1
    elif split == "tile":
        split_size = 64
        num_splits = max(1, -(-longest // 64))
    elif split == "ref20":                      # the reference's default split size (src/gemma4.h:24)
        split_size = 20
        num_splits = max(1, -(-longest // 20))
    else:
        split_size = 37
        num_splits = max(1, -(-longest // 37)) + 5
    d = DeviceCase(kv, case)
    out, lse, pm = d.run(split_size, num_splits, poison=float("nan"))
    check(orc, case, out, lse)
    if pm is not None and split_size > 0:
        for b, n in enumerate(live_keys(case)):
            actual = -(-n // split_size)
            assert not np.isnan(pm[b, :, :actual]).any()
            assert np.isnan(pm[b, :, actual:]).all()          # dead splits never touch the scratch


def test_unmapped_pages_and_empty_rows(kv, orc):
    case = make_attn_case(13, [100, 0, 40, 64], window=0)
    case.page_table[0, 2] = -1
    case.page_table[2, 0] = case.cfg[1] + 5
    case.page_table[3, :] = -1                      # every page of sequence 3 unmapped
    d = DeviceCase(kv, case)
    for split_size, num_splits in ((128, 1), (16, 7), (16, 12), (8, 13)):
        out, lse, _ = d.run(split_size, num_splits)
        check(orc, case, out, lse)
        assert not out[1].any() and not out[3].any()
        assert np.isneginf(lse[1]).all() and np.isneginf(lse[3]).all()


def test_balanced_partition_edge_cases(kv, orc):
    """split_size == 0: ranges cut sequences anywhere, skip empty and unmapped ones, and a scratch that
    only allows a few CTAs still gives the same answer."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    case = make_attn_case(77, [100, 0, 40, 64, 3000, 1, 0, 517], window=0)
    case.page_table[0, 2] = -1
    case.page_table[3, :] = -1
    d = DeviceCase(kv, case)
    for num_splits in (kv.plan_balanced(case.batch, sms), 2, 3, 9):
        out, lse, _ = d.run(0, num_splits, poison=float("nan"))
        check(orc, case, out, lse)
        assert not out[1].any() and not out[3].any() and not out[6].any()
    ring = make_attn_case(78, [5000, 90, 1024, 1023, 1025, 0, 2000], window=1024)
    d = DeviceCase(kv, ring)
    for num_splits in (kv.plan_balanced(ring.batch, sms), 2):
        out, lse, _ = d.run(0, num_splits, poison=float("nan"))
        check(orc, ring, out, lse)
    many = make_attn_case(79, list(np.random.default_rng(3).integers(0, 40, size=300)), window=0)
    out, lse, _ = DeviceCase(kv, many).run(0, kv.plan_balanced(many.batch, sms), poison=float("nan"))
    check(orc, many, out, lse)
    # rejected: scratch too small for even one CTA, or a geometry the balanced kernel is not built for
    small = make_attn_case(80, [64, 64], window=0)
    d = DeviceCase(kv, small)
    B, H, D = 2, 16, 256
    buf = torch.zeros(B * H * D, dtype=torch.float32, device="cuda")
    args = (torch.zeros((B, H, D), dtype=torch.int16, device="cuda"), None, d.q, d.ck, d.cv, d.cfg, d.table, d.seq,
            0, small.scale, 0, 1, B, H, buf, buf, buf)
    assert kv.decode_attention(*args, check=False) == kv.CUDA_ERROR_INVALID_VALUE
    kv4 = make_attn_case(81, [64], window=0, kv_heads=4, q_heads=8)
    d4 = DeviceCase(kv, kv4)
    assert kv.decode_attention(torch.zeros((1, 8, 256), dtype=torch.int16, device="cuda"), None, d4.q, d4.ck, d4.cv,
                               d4.cfg, d4.table, d4.seq, 0, kv4.scale, 0, 8, 1, 8, buf, buf, buf,
                               check=False) == kv.CUDA_ERROR_INVALID_VALUE


def test_all_sequences_empty(kv, orc):
    case = make_attn_case(14, [0, 0], window=0)
    d = DeviceCase(kv, case)
    for split_size, num_splits in ((16, 1), (16, 3), (0, 200)):
        out, lse, _ = d.run(split_size, num_splits)
        assert not out.any() and np.isneginf(lse).all()


def test_lse_optional_and_stale_scratch_is_ignored(kv, orc):
    case = make_attn_case(15, [333, 40], window=0)
    d = DeviceCase(kv, case)
    out_a, _, _ = d.run(32, 11, poison=1.0e30, want_lse=False)
    out_b, _, _ = d.run(32, 11, poison=-7.0)
    assert np.array_equal(out_a, out_b)
    check(orc, case, out_a, None)


def test_uniform_scores_give_the_mean_and_log_count(kv, orc):
    """K = 0 makes every score 0: the output is the mean of the live V rows and LSE = ln(live keys),
    whatever the split geometry (a size-independent property of the path)."""
    case = make_attn_case(16, [777, 1500], window=1024)
    case.cache_k[:] = 0
    d = DeviceCase(kv, case)
    for split_size, num_splits in ((1024, 1), (64, 16), (24, 50), (0, 160)):
        out, lse, _ = d.run(split_size, num_splits)
        for b, n in enumerate(live_keys(case)):
            assert np.abs(lse[b] - math.log(n)).max() <= 1e-4
        check(orc, case, out, lse)


def test_page_pool_permutation_invariance(kv, orc):
    """Re-laying the same logical pages over other physical pages leaves the output bit-identical."""
    case = make_attn_case(18, [1500, 260, 33], window=0, extra_pages=9)
    d = DeviceCase(kv, case)
    out_a, lse_a, _ = d.run(64, 24)
    cfg = case.cfg
    page_elems = cfg[2] * cfg[5] * cfg[6]
    perm = np.random.default_rng(5).permutation(cfg[1])          # new physical index of old page p is perm[p]
    k2 = np.empty_like(case.cache_k); v2 = np.empty_like(case.cache_v)
    k2.reshape(cfg[1], page_elems)[perm] = case.cache_k.reshape(cfg[1], page_elems)
    v2.reshape(cfg[1], page_elems)[perm] = case.cache_v.reshape(cfg[1], page_elems)
    table2 = np.where(case.page_table >= 0, perm[np.maximum(case.page_table, 0)], -1).astype(np.int32)
    case2 = make_attn_case(18, [1500, 260, 33], window=0, extra_pages=9)
    case2.cache_k, case2.cache_v, case2.page_table = k2, v2, table2
    out_b, lse_b, _ = DeviceCase(kv, case2).run(64, 24)
    assert np.array_equal(out_a, out_b) and np.array_equal(lse_a, lse_b)


def test_layer_step_append_then_attend(kv, orc):
    """One layer-step through b200kv_decode_layer_step_bf16 on config 1: 1024 tokens already in a tight
    ring, append position 1024 (overwrites slot 0 / offset 0), attend over keys 1..1024."""
    import ctypes
    from tests.helpers import make_append_case
    acase = make_append_case(31, [1024], window=1024, ring_pages=64, max_pos=1025)
    case = make_attn_case(32, [1025], window=1024, ring_pages=64, permute=False)
    case.page_table = acase.page_table.copy()
    cfg = kv.make_kv_config(*acase.cfg)
    assert acase.cfg == case.cfg
    ck, cv = case.cache_k.copy(), case.cache_v.copy()
    dck, dcv = dev(ck), dev(cv)
    B, H, D = 1, 16, 256
    split_size, num_splits = kv.plan_splits(1, 1024, 8, 148)
    dq = torch.zeros((B, H, D), dtype=torch.int16, device="cuda")
    out = torch.zeros_like(dq)
    lse = torch.zeros((B, H), dtype=torch.float32, device="cuda")
    pm = torch.zeros(B * H * num_splits, dtype=torch.float32, device="cuda"); pl = torch.zeros_like(pm)
    pacc = torch.zeros(B * H * num_splits * D, dtype=torch.float32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    keep = [dev(acase.q), dev(acase.k), dev(acase.v), dev(acase.q_w), dev(acase.k_w), dev(acase.cos), dev(acase.sin),
            dev(acase.page_table), dev(acase.token_position), dev(case.seq_lengths)]
    a = kv.LayerStepArgs()
    a.q, a.out, a.lse = dq.data_ptr(), out.data_ptr(), lse.data_ptr()
    a.partial_m, a.partial_l, a.partial_acc = pm.data_ptr(), pl.data_ptr(), pacc.data_ptr()
    a.cache_k, a.cache_v, a.cache_config = dck.data_ptr(), dcv.data_ptr(), cfg
    a.page_table, a.token_position, a.seq_lengths = keep[7].data_ptr(), keep[8].data_ptr(), keep[9].data_ptr()
    a.cache_layer, a.split_size, a.num_splits, a.softmax_scale = 0, split_size, num_splits, 1.0 / 16.0
    a.raw_q, a.raw_k, a.raw_v = keep[0].data_ptr(), keep[1].data_ptr(), keep[2].data_ptr()
    a.q_norm_weight, a.k_norm_weight, a.cos, a.sin = (keep[3].data_ptr(), keep[4].data_ptr(),
                                                      keep[5].data_ptr(), keep[6].data_ptr())
    a.batch_count, a.q_heads, a.rotary_dim, a.norm_mode = 1, 16, 256, kv.NORM_IEEE
    a.status = status.data_ptr()
    kv.decode_layer_step(a)
    torch.cuda.synchronize()
    assert status[0].item() == 0
    qp = np.zeros((B, H, D), dtype=np.uint16)
    orc.decode_append(qp, ck, cv, acase.cfg, acase.page_table, acase.token_position, 0, acase.q, acase.k, acase.v,
                      acase.q_w, acase.k_w, acase.cos, acase.sin, 1, 16, 256)
    assert np.array_equal(host_u16(dck), ck) and np.array_equal(host_u16(dcv), cv)     # cache state bit-exact
    assert np.array_equal(host_u16(dq), qp.reshape(-1))
    ref, ref_lse = orc.decode_attention_f64(qp, ck, cv, acase.page_table, case.seq_lengths, acase.cfg, 0, 1 / 16.0, 1, 16)
    max_abs, max_rel = attention_error(host_u16(out), ref)
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL
    assert np.abs(lse.cpu().numpy() - ref_lse).max() <= LSE_MAX_ABS


def test_bounded_wait_reports_instead_of_hanging(kv, orc):
    """The status word of a normal run stays 0. Then the give-up path every kernel shares is seen to run:
    b200kv_bounded_wait_selftest has one warp wait, with the library's bounded mbarrier wait, on a barrier nothing
    arrives at, for 2^20 / 2^23 SM clocks; it must write B200KV_STATUS_WAIT_TIMEOUT, have waited at least the
    limit and not much longer (the clock is read every 64 polls, each of which may park the warp for a while), and return normally -- after which the same attention call gives the same bits and
    a clean status again. Nothing faults, traps or hangs."""
    case = make_attn_case(40, [256], window=0)
    d = DeviceCase(kv, case)
    first, _, _ = d.run(64, 4)                    # asserts a clean status itself
    word = torch.zeros(4, dtype=torch.int32, device="cuda")
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    for limit in (1 << 20, 1 << 23):
        word.zero_()
        kv.bounded_wait_selftest(limit, word, waited)
        torch.cuda.synchronize()
        assert word[0].item() == kv.STATUS_WAIT_TIMEOUT
        assert limit < waited.item() < limit + (1 << 22), waited.item()
    assert kv.bounded_wait_selftest(0, word, waited, check=False) == 1            # limits outside 1 .. 2^28 are refused
    assert kv.bounded_wait_selftest(1 << 40, word, waited, check=False) == 1
    again, _, _ = d.run(64, 4)
    assert np.array_equal(again, first)


@pytest.mark.parametrize("name,seq_lens,window,kvh,dim,split", [
    ("balanced batch 1 ring", [1500], 1024, 8, 256, 0),
    ("balanced ragged", [700, 33, 1500, 64, 260, 1024, 2000, 90], 0, 8, 256, 0),
    ("fixed splits, 2 KV heads", [3000, 70, 1024, 513], 0, 2, 256, 128),
    ("16 query heads on one KV head of 512", [4096], 0, 1, 512, 0),
])
def test_launches_back_to_back_give_the_same_bits(kv, name, seq_lens, window, kvh, dim, split):
    """300 launches enqueued without a host synchronisation in between (each may start under its predecessor's
    tail: programmatic dependent launch) on the same inputs and the same scratch: every output the first one's
    bits, no wait running out."""
    hq = 16 if kvh in (8, 1) else 2 * kvh
    case = make_attn_case(11, seq_lens, window=window, kv_heads=kvh, q_heads=hq, head_dim=dim)
    B = len(seq_lens)
    cfg = kv.make_kv_config(*case.cfg)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    live = max(min(s, window) if window else s for s in seq_lens)
    ns = kv.plan_balanced(B, sms) if split == 0 else -(-live // split)
    d = [dev(x) for x in (case.q, case.cache_k, case.cache_v, case.page_table, case.seq_lengths)]
    pm = torch.zeros(B * hq * ns, device="cuda")
    pl, pacc = pm.clone(), torch.zeros(B * hq * ns * dim, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    outs = []
    for _ in range(300):
        out = torch.full((B, hq, dim), 0x7FC0, dtype=torch.int16, device="cuda")
        lse = torch.zeros(B, hq, device="cuda")
        kv.decode_attention(out, lse, d[0], d[1], d[2], cfg, d[3], d[4], 0, case.scale, split, ns, B, hq, pm, pl, pacc,
                            status)
        outs.append((out, lse))
    torch.cuda.synchronize()
    assert status[0].item() == 0
    for out, lse in outs[1:]:
        assert torch.equal(out, outs[0][0]) and torch.equal(lse, outs[0][1]), name
