"""Internal consistency of the CPU oracle: independent restatements of the same math agree,
and the edge cases of the path behave as the reference source says they do."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from tests import helpers
from tests.helpers import ATTN_MAX_ABS, ATTN_MAX_REL, attention_error, make_append_case, make_attn_case


def test_bf16_round_trip_matches_torch(orc):
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.standard_normal(4096).astype(np.float32) * 3.0,
        np.array([0.0, -0.0, 1.0, np.inf, -np.inf, 1e-40, 3.3895314e38, np.nan], dtype=np.float32),
        (np.arange(1 << 16, dtype=np.uint32) << 15).view(np.float32),   # every tie and near-tie pattern
    ])
    got = orc.f32_to_bf16(x)
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    nan = np.isnan(x)
    assert np.array_equal(got[~nan], want[~nan])
    assert np.all(got[nan] == 0x7FFF)           # __float2bfloat16_rn's canonical NaN


def test_e4m3_codec_matches_torch(orc):
    codes = np.arange(256, dtype=np.uint8)
    dec = orc.e4m3_to_f32(codes)
    want = torch.from_numpy(codes).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    finite = ~np.isnan(want)
    assert np.array_equal(dec[finite], want[finite]) and np.all(np.isnan(dec[~finite]))
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s for s in (1e-3, 0.1, 1.0, 30.0, 200.0)])
    x = np.concatenate([x, dec[finite], np.float32([447.9, 448.0, 463.9, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10])])
    inside = np.abs(x) <= 448.0
    got = np.array([orc.lib().orc_f32_to_e4m3(float(v)) for v in x[inside]], dtype=np.uint8)
    want_codes = torch.from_numpy(x[inside]).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(got, want_codes)
    # saturating finite conversion beyond the largest normal
    for v, code in ((1000.0, 0x7E), (-1000.0, 0xFE), (float("inf"), 0x7E), (464.0, 0x7E), (-500.0, 0xFE)):
        assert orc.lib().orc_f32_to_e4m3(v) == code


def _numpy_prep(x_bf16, w_bf16, cos_row, sin_row, rotary_dim, orc):
    """Straightforward double-precision RMSNorm + split-half RoPE (order-free restatement)."""
    x = orc.bf16_to_f32(x_bf16).astype(np.float64)
    D = x.size
    scale = 1.0 / math.sqrt((x * x).sum() / D + 1e-6)
    t = x * scale * (orc.bf16_to_f32(w_bf16).astype(np.float64) if w_bf16 is not None else 1.0)
    out = t.copy()
    half = rotary_dim // 2
    if cos_row is not None:
        lo, hi = t[:half], t[half:rotary_dim]
        out[:half] = lo * cos_row - hi * sin_row
        out[half:rotary_dim] = lo * sin_row + hi * cos_row
    return out


@pytest.mark.parametrize("head_dim,rotary_dim", [(256, 256), (512, 128)])
def test_prep_within_one_bf16_ulp_of_double(orc, head_dim, rotary_dim):
    rng = np.random.default_rng(7)
    cos, sin = orc.fill_rope_tables(50, rotary_dim // 2, 10000.0, head_dim)
    for trial in range(8):
        x = helpers.bf16_normal(rng, (head_dim,), std=float(rng.uniform(0.1, 4.0)))
        w = helpers.bf16_normal(rng, (head_dim,), std=0.05, mean=1.0)
        pos = int(rng.integers(0, 50))
        got = orc.bf16_to_f32(orc.prep_weighted_rope_head(x, w, cos[pos].copy(), sin[pos].copy(), rotary_dim))
        want = _numpy_prep(x, w, cos[pos].astype(np.float64), sin[pos].astype(np.float64), rotary_dim, orc)
        ulp = np.maximum(np.abs(want), 2.0 ** -120) * 2.0 ** -7
        assert np.all(np.abs(got - want) <= ulp)
        got_v = orc.bf16_to_f32(orc.prep_scale_free_head(x))
        want_v = _numpy_prep(x, None, None, None, rotary_dim, orc)
        assert np.all(np.abs(got_v - want_v) <= np.maximum(np.abs(want_v), 2.0 ** -120) * 2.0 ** -7)


def test_zero_row_preps_to_zero(orc):
    x = np.zeros(256, dtype=np.uint16)
    w = orc.f32_to_bf16(np.ones(256, dtype=np.float32))
    cos, sin = orc.fill_rope_tables(4, 128, 10000.0, 256)
    assert not orc.prep_weighted_rope_head(x, w, cos[3].copy(), sin[3].copy(), 256).astype(np.uint16).view(np.int16).any() \
        or np.all(orc.bf16_to_f32(orc.prep_weighted_rope_head(x, w, cos[3].copy(), sin[3].copy(), 256)) == 0.0)
    assert np.all(orc.bf16_to_f32(orc.prep_scale_free_head(x)) == 0.0)


def test_append_places_rows_and_wraps_the_ring(orc):
    """Config 1: tight ring of 64 x 16 = 1024 tokens; position 1024 lands on slot 0 offset 0."""
    case = make_append_case(3, [1024], page_size=16, window=1024, ring_pages=64, max_pos=1025)
    cfg = case.cfg
    elems = cfg[0] * cfg[1] * cfg[2] * cfg[5] * cfg[6]
    ck = np.full(elems, 0x1234, dtype=np.uint16)
    cv = np.full(elems, 0x4321, dtype=np.uint16)
    qp = np.zeros_like(case.q)
    orc.decode_append(qp, ck, cv, cfg, case.page_table, case.token_position, 0, case.q, case.k, case.v,
                      case.q_w, case.k_w, case.cos, case.sin, 1, 16, 256)
    phys = case.page_table[0, 0]
    base = orc.cache_offset(cfg, 0, int(phys), 0, 0, 0)
    row = cfg[5] * cfg[6]
    assert not np.any(ck[base:base + row] == 0x1234)
    untouched = np.ones(elems, dtype=bool)
    untouched[base:base + row] = False
    assert np.all(ck[untouched] == 0x1234) and np.all(cv[untouched] == 0x4321)
    # rows equal the stand-alone prep of the same heads
    for h in range(8):
        want = orc.prep_weighted_rope_head(case.k[0, h].copy(), case.k_w, case.cos[1024].copy(),
                                           case.sin[1024].copy(), 256)
        assert np.array_equal(ck[base + h * 256: base + (h + 1) * 256], want)
        assert np.array_equal(cv[base + h * 256: base + (h + 1) * 256], orc.prep_scale_free_head(case.v[0, h].copy()))
    assert qp.any()


def test_write_guards(orc):
    """src/gemma4_kv_cache.cu:27-34: negative batch/position, batch out of range, linear capacity and
    unmapped or out-of-pool pages all drop the row; a ring wraps instead."""
    cfg = (1, 4, 4, 2, 2, 2, 16, 0)         # linear, capacity 8 tokens per sequence
    table = np.array([[0, 1], [9, -1]], dtype=np.int32)      # 9 is outside the pool
    tb = np.array([0, 0, -1, 0, 2, 1, 1, 0], dtype=np.int32)
    tp = np.array([0, 5, 1, -3, 0, 0, 4, 8], dtype=np.int32)  # last: logical page 2 >= 2 -> dropped
    rng = np.random.default_rng(5)
    k = helpers.bf16_normal(rng, (tb.size, 2, 16))
    v = helpers.bf16_normal(rng, (tb.size, 2, 16))
    elems = 4 * 4 * 2 * 16
    ck, cv = np.zeros(elems, dtype=np.uint16), np.zeros(elems, dtype=np.uint16)
    assert orc.kv_cache_write(ck, cv, cfg, table, tb, tp, 0, k, v) == 0
    want = np.zeros(elems, dtype=np.uint16)
    want[0:32] = k[0].reshape(-1)                       # page 0 offset 0
    off = orc.cache_offset(cfg, 0, 1, 1, 0, 0)          # position 5 -> page slot 1 offset 1
    want[off:off + 32] = k[1].reshape(-1)
    assert np.array_equal(ck, want)
    ring = (1, 4, 4, 2, 2, 2, 16, 8)
    ck2, cv2 = np.zeros(elems, dtype=np.uint16), np.zeros(elems, dtype=np.uint16)
    assert orc.kv_cache_write(ck2, cv2, ring, table, tb[-1:], tp[-1:], 0, k[-1:], v[-1:]) == 0
    assert np.array_equal(ck2[0:32], k[-1].reshape(-1))     # position 8 wraps to slot 0 offset 0
    assert orc.kv_cache_write(ck, cv, cfg, table, tb, tp, 3, k, v) != 0   # bad layer -> invalid value


CASES = [
    dict(seq_lens=[1025], window=1024, ring_pages=64),            # config 1 (tight ring, wrapped)
    dict(seq_lens=[1041], window=1024),                           # slack ring past its wrap point
    dict(seq_lens=[300, 17, 1, 64, 129], window=0),               # mixed lengths, linear
    dict(seq_lens=[5], window=0),
    dict(seq_lens=[700, 90], window=256, ring_pages=20, page_size=16),
    dict(seq_lens=[200], window=0, page_size=64),
    dict(seq_lens=[77, 31], window=0, page_size=4),
    dict(seq_lens=[150], window=0, kv_heads=1, q_heads=16, head_dim=512),   # reference-native global
    dict(seq_lens=[400], window=0, outlier_frac=0.05),
]


@pytest.mark.parametrize("kw", CASES)
@pytest.mark.parametrize("split_size,slack", [(20, 0), (64, 3), (10 ** 6, 0)])
def test_reference_order_attention_within_tolerance_of_double(orc, kw, split_size, slack):
    case = make_attn_case(11, **kw)
    live = [min(int(s), kw.get("window") or int(s)) for s in case.seq_lengths]
    num_splits = max(1, -(-max(live) // split_size)) + slack
    out64, lse = orc.decode_attention_f64(case.q, case.cache_k, case.cache_v, case.page_table, case.seq_lengths,
                                          case.cfg, 0, case.scale, case.batch, case.q_heads)
    out, pm, pl, pacc = orc.decode_attention_ref(case.q, case.cache_k, case.cache_v, case.page_table,
                                                 case.seq_lengths, case.cfg, 0, case.scale, split_size,
                                                 num_splits, case.batch, case.q_heads, poison=np.nan)
    max_abs, max_rel = attention_error(out, out64)
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL
    if num_splits > 1:
        # over-provisioned splits leave the (poisoned) scratch untouched (decode.cu:746-748)
        pm = pm.reshape(case.batch, case.q_heads, num_splits)
        for b, n in enumerate(live):
            actual = -(-n // split_size)
            assert not np.isnan(pm[b, :, :actual]).any()
            assert np.isnan(pm[b, :, actual:]).all()


def test_unmapped_pages_and_empty_rows(orc):
    case = make_attn_case(13, [100, 0, 40], window=0)
    case.page_table[0, 2] = -1                    # keys 32..47 of sequence 0 vanish
    case.page_table[2, 0] = case.cfg[1] + 5       # beyond the pool: skipped too
    out64, lse = orc.decode_attention_f64(case.q, case.cache_k, case.cache_v, case.page_table, case.seq_lengths,
                                          case.cfg, 0, case.scale, 3, 16)
    assert np.all(out64[1] == 0.0) and np.all(np.isneginf(lse[1]))     # seq_len 0 -> zeros
    for split_size, num_splits in ((1000, 1), (16, 7), (16, 12)):
        out, *_ = orc.decode_attention_ref(case.q, case.cache_k, case.cache_v, case.page_table, case.seq_lengths,
                                           case.cfg, 0, case.scale, split_size, num_splits, 3, 16)
        assert not np.isnan(orc.bf16_to_f32(out)).any()
        assert np.all(out[1] == 0)
        max_abs, max_rel = attention_error(out, out64)
        assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL
    # a sequence whose every page is unmapped has no attention mass: zeros, never NaN (decode.cu:684,856,972)
    case.page_table[2, :] = -1
    out, *_ = orc.decode_attention_ref(case.q, case.cache_k, case.cache_v, case.page_table, case.seq_lengths,
                                       case.cfg, 0, case.scale, 16, 7, 3, 16)
    assert np.all(out[2] == 0)


def test_window_counts_the_current_token(orc):
    """src/gemma4.h:22-23: live keys are [seq_len - window, seq_len)."""
    case = make_attn_case(17, [50], window=32, ring_pages=3, page_size=16)
    out64, lse = orc.decode_attention_f64(case.q, case.cache_k, case.cache_v, case.page_table, case.seq_lengths,
                                          case.cfg, 0, case.scale, 1, 16)
    # recompute by hand over positions 18..49 through the ring addressing
    D, H = 256, 8
    kf = orc.bf16_to_f32(case.cache_k)
    qf = orc.bf16_to_f32(case.q)[0]
    scores = []
    for pos in range(18, 50):
        slot = (pos // 16) % 3
        base = orc.cache_offset(case.cfg, 0, int(case.page_table[0, slot]), pos % 16, 0, 0)
        scores.append(float(np.dot(kf[base:base + D].astype(np.float64), qf[0].astype(np.float64))) * case.scale)
    want = math.log(np.exp(np.array(scores) - max(scores)).sum()) + max(scores)
    assert abs(lse[0, 0] - want) <= 1e-4


def test_fp8_append_rule(orc):
    """Scale grows monotonically inside a page, earlier rows are requantised when it grows, a new
    page (offset 0) starts from its own first row, and bulk == incremental only when no growth happens."""
    cfg = (1, 3, 16, 3, 1, 2, 256, 0)
    table = np.array([[2, 0, 1]], dtype=np.int32)
    rng = np.random.default_rng(23)
    n = 40
    k = helpers.bf16_normal(rng, (n, 2, 256))
    v = helpers.bf16_normal(rng, (n, 2, 256))
    k[5] = orc.f32_to_bf16(orc.bf16_to_f32(k[5]) * 6.0)     # forces a scale jump at offset 5
    elems = 3 * 16 * 2 * 256
    ck, cv = np.zeros(elems, dtype=np.uint8), np.zeros(elems, dtype=np.uint8)
    sk, sv = np.zeros(6, dtype=np.float32), np.zeros(6, dtype=np.float32)
    prev = None
    for t in range(n):
        orc.fp8_append(ck, cv, sk, sv, cfg, table, np.array([0], np.int32), np.array([t], np.int32),
                       np.array([1], np.int32), 0, np.ascontiguousarray(k[t:t + 1]), np.ascontiguousarray(v[t:t + 1]))
        page = int(table[0, t // 16])
        if t % 16 and prev is not None:
            assert np.all(sk[page * 2:(page + 1) * 2] >= prev)
        prev = sk[page * 2:(page + 1) * 2].copy()
    # dequantised rows stay close to the source: |x - dec * s| <= s * 2^-3 * |code| quantum bound ~ 1/16 rel
    kd = orc.e4m3_to_f32(orc.fp8_k_rows(ck, cfg)[0])          # [page, token, head, dim]
    assert orc.lib().orc_fp8_k_index(__import__("ctypes").byref(orc.OrcKvConfig.of(cfg)), 0, 1, 9, 1, 37) == \
        1 * 16 * 2 * 256 + 1 * 8 * 2 * 256 + 1 * 8 * 256 + 1 * 256 + ((2 ^ 4) * 16 + 5)
    for t in range(n):
        page = int(table[0, t // 16])
        for h in range(2):
            deq = kd[page, t % 16, h] * sk[page * 2 + h]
            src = orc.bf16_to_f32(k[t, h])
            assert np.abs(deq - src).max() <= 0.13 * np.abs(src).max() + 1e-6
    # amax row of every page maps to +-448 exactly
    amax_code = np.abs(kd).reshape(3, 16, 2, 256).max(axis=(1, 3))
    assert np.all(amax_code[[2, 0]] == 448.0)
    # one bulk call over the same rows gives the same scales (max is order-free)
    ck2, cv2 = np.zeros(elems, dtype=np.uint8), np.zeros(elems, dtype=np.uint8)
    sk2, sv2 = np.zeros(6, dtype=np.float32), np.zeros(6, dtype=np.float32)
    orc.fp8_append(ck2, cv2, sk2, sv2, cfg, table, np.array([0], np.int32), np.array([0], np.int32),
                   np.array([n], np.int32), 0, k, v)
    assert np.array_equal(sk, sk2) and np.array_equal(sv, sv2)
    # V never had a jump large enough to double-round beyond one code step
    assert np.abs(orc.e4m3_to_f32(cv).astype(np.float32) - orc.e4m3_to_f32(cv2)).max() <= 64.0
