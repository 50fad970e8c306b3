"""Pins the CPU oracle to the cases the reference's own tests hold for this path.

Each test restates one case of the reference's test executables (closed-form
inputs, expected values and tolerances as written there) and requires the
oracle to meet it. The reference has no numerical test of the decode
split/reduce phases or of the fused decode append; those are pinned by the
golden fixtures recorded from the reference's CUDA kernels (tests/golden).
"""
from __future__ import annotations

import math

import numpy as np

from tests.helpers import closed_form_value


def test_invalid_page_write_is_a_noop(orc):
    """tests/test_kv_cache.cu:94-133: token_batch=1 >= batch_size=1 and an all -1 page
    table must leave both caches all-zero (tolerance 0)."""
    cfg = (1, 2, 4, 2, 1, 2, 16, 0)
    page_table = np.full(cfg[3], -1, dtype=np.int32)
    token_batch = np.array([1], dtype=np.int32)
    token_position = np.array([0], dtype=np.int32)
    n = cfg[5] * cfg[6]
    k = closed_form_value(43000 + np.arange(n))
    v = closed_form_value(44000 + np.arange(n))
    elems = cfg[0] * cfg[1] * cfg[2] * cfg[5] * cfg[6]
    cache_k = np.zeros(elems, dtype=np.uint16)
    cache_v = np.zeros(elems, dtype=np.uint16)
    assert orc.kv_cache_write(cache_k, cache_v, cfg, page_table, token_batch, token_position, 0, k, v) == 0
    assert not cache_k.any() and not cache_v.any()


def test_runtime_prefill_then_decode_metadata(orc):
    """tests/test_runtime_state.cu:29-107."""
    rt = orc.Runtime(2, 66, 64)
    assert rt.prepare_prefill(64) == 0
    sliding, glob, token_count = rt.configs()
    assert token_count == 128
    assert list(rt.array("seq_lengths")) == [64, 64]
    tb, tp = rt.array("token_batch"), rt.array("token_position")
    assert (tb[63], tp[63], tb[64], tp[64]) == (0, 63, 1, 0)   # batch-major rows
    st, gt = rt.array("sliding_page_table"), rt.array("global_page_table")
    assert st[0] >= 0 and st[sliding.max_pages_per_seq] >= 0
    assert gt[0] >= 0 and gt[glob.max_pages_per_seq] >= 0

    assert rt.prepare_decode_step() == 0
    _, _, token_count = rt.configs()
    assert token_count == 2
    assert list(rt.array("seq_lengths")) == [65, 65]
    assert list(rt.array("token_batch")[:2]) == [0, 1]
    assert list(rt.array("token_position")[:2]) == [64, 64]
    assert rt.array("sliding_page_table")[1] == 1 and rt.array("global_page_table")[1] == 1

    # A step that must fail (66 >= max_seq_len) mutates nothing.
    rt.array("seq_lengths")[:] = [64, 66]
    names = ["seq_lengths", "token_batch", "token_position", "sliding_page_table", "global_page_table",
             "sliding_slot_logical_pages", "global_slot_logical_pages"]
    before = {n: rt.array(n).copy() for n in names}
    assert rt.prepare_decode_step() != 0
    for n in names:
        assert np.array_equal(rt.array(n), before[n]), n


def test_runtime_prep_smoke(orc):
    """tests/test_decode_megakernel.cu:16-40."""
    rt = orc.Runtime(1, 4, 2)
    assert rt.prepare_prefill(2) == 0
    assert rt.configs()[2] == 2 and rt.array("seq_lengths")[0] == 2
    assert rt.prepare_decode_step() == 0
    assert rt.configs()[2] == 1 and rt.array("seq_lengths")[0] == 3


def test_rope_tables(orc):
    """tests/test_runtime_state.cu:110-140: sliding cos/sin at (pos 1, i 0) are cos(1), sin(1);
    global (theta 1e6, exponent over 512, 64 pairs) at (pos 1, i 1) to 1e-6."""
    cos, sin = orc.fill_rope_tables(4, 128, 10000.0, 256)
    assert abs(cos[1, 0] - math.cos(1.0)) <= 1e-6
    assert abs(sin[1, 0] - math.sin(1.0)) <= 1e-6
    gcos, _ = orc.fill_rope_tables(4, 64, 1000000.0, 512)
    expected = math.cos(np.float32(1000000.0) ** np.float32(-2.0 / 512.0))
    assert abs(gcos[1, 1] - expected) <= 1e-6


def _global_prep_case(orc):
    """Inputs of tests/test_flash_attention.cu:232-346 (global 1 KV x 512, rotary 128,
    unit weights, positions {2, 4}, hand-set cos/sin at those positions)."""
    D, half, rows = 512, 64, 2
    k = closed_form_value(110000 + np.arange(rows * D)).reshape(rows, 1, D)
    q = np.zeros((rows, 16, D), dtype=np.uint16)
    w = orc.f32_to_bf16(np.ones(D, dtype=np.float32))
    pos = np.array([2, 4], dtype=np.int32)
    cos = np.ones((5, half), dtype=np.float32)
    sin = np.zeros((5, half), dtype=np.float32)
    cos[2, 0], sin[2, 0] = 0.0, 1.0
    cos[4, 0], sin[4, 0] = 0.0, -1.0
    return D, half, rows, q, k, w, pos, cos, sin


def test_global_prep_k_derived_v_and_absolute_position_rope(orc):
    D, half, rows, q, k, w, pos, cos, sin = _global_prep_case(orc)
    qp, kp, vp = orc.prefill_prep(q, k, None, w, w, cos, sin, pos, 16, 1, D, 128)
    kf = orc.bf16_to_f32(k).reshape(rows, D)
    # expected as the test computes it: plain fp32 running sum, 1/sqrt(mean + eps)
    inv_rms = np.empty(rows, dtype=np.float32)
    for r in range(rows):
        s = np.float32(0.0)
        for d in range(D):
            s = np.float32(s + kf[r, d] * kf[r, d])
        inv_rms[r] = np.float32(1.0) / np.sqrt(np.float32(s / np.float32(D)) + np.float32(1e-6))
    expected_v = orc.bf16_to_f32(orc.f32_to_bf16(kf * inv_rms[:, None]))
    got_v = orc.bf16_to_f32(vp).reshape(rows, D)
    assert np.abs(got_v - expected_v).max() <= 0.00390625  # 2^-8, :299
    got_k = orc.bf16_to_f32(kp).reshape(rows, D)
    for r in range(rows):
        c, s = cos[pos[r], 0], sin[pos[r], 0]
        lo, hi = kf[r, 0] * inv_rms[r], kf[r, half] * inv_rms[r]
        exp_lo = orc.bf16_to_f32(orc.f32_to_bf16(np.float32(lo * c - hi * s)))
        exp_hi = orc.bf16_to_f32(orc.f32_to_bf16(np.float32(lo * s + hi * c)))
        assert abs(got_k[r, 0] - exp_lo) <= 0.00390625   # :319-324
        assert abs(got_k[r, half] - exp_hi) <= 0.00390625


def test_global_uniform_attention_rows(orc):
    """Same case, attention part (:326-345): q = 0 gives uniform weights, so the row that sees
    one key returns v0 and the row that sees two returns (v0 + v1) / 2, tolerance 2^-5. The decode
    oracle is asked for exactly those two rows (seq_len 1 and 2 over the same cache)."""
    D, half, rows, q, k, w, pos, cos, sin = _global_prep_case(orc)
    qp, kp, vp = orc.prefill_prep(q, k, None, w, w, cos, sin, pos, 16, 1, D, 128)
    cfg = (1, 1, 2, 1, 1, 1, D, 0)           # one page of two tokens
    page_table = np.zeros((1, 1), dtype=np.int32)
    vf = orc.bf16_to_f32(vp).reshape(rows, D)
    for seq_len, expected in ((1, vf[0]), (2, 0.5 * (vf[0] + vf[1]))):
        seq = np.array([seq_len], dtype=np.int32)
        qrow = np.ascontiguousarray(qp[seq_len - 1:seq_len])
        for split_size, num_splits in ((64, 1), (1, 2)):
            out, *_ = orc.decode_attention_ref(qrow, kp.reshape(-1), vp.reshape(-1), page_table, seq, cfg, 0,
                                               1.0 / math.sqrt(D), split_size, num_splits, 1, 16)
            got = orc.bf16_to_f32(out).reshape(16, D)
            assert np.abs(got - expected[None, :]).max() <= 0.03125
        out64, lse = orc.decode_attention_f64(qrow, kp.reshape(-1), vp.reshape(-1), page_table, seq, cfg, 0,
                                              1.0 / math.sqrt(D), 1, 16)
        assert np.abs(out64.reshape(16, D) - expected[None, :]).max() <= 0.03125
        assert np.allclose(lse, math.log(seq_len), atol=1e-6)


def test_attention_matches_the_reference_tests_cpu_formula(orc):
    """tests/test_flash_attention.cu:118-172: scores in fp32 running sums, exp(score - max),
    output sum((w / denom) * v). Its last causal row equals a decode over the same keys;
    tolerance 2^-5 as the test states (:227)."""
    D, seq_len, q_heads = 512, 33, 16
    q = closed_form_value(4000 + np.arange(seq_len * q_heads * D), 29, 11, 512.0).reshape(seq_len, q_heads, D)
    k = closed_form_value(5000 + np.arange(seq_len * D), 29, 11, 512.0).reshape(seq_len, 1, D)
    w = orc.f32_to_bf16(np.ones(D, dtype=np.float32))
    cos = np.ones((seq_len, 64), dtype=np.float32)
    sin = np.zeros((seq_len, 64), dtype=np.float32)
    pos = np.arange(seq_len, dtype=np.int32)
    qp, kp, vp = orc.prefill_prep(q, k, None, w, w, cos, sin, pos, q_heads, 1, D, 128)
    scale = np.float32(1.0 / math.sqrt(D))
    qf = orc.bf16_to_f32(qp)[seq_len - 1]               # [16, 512]
    kf = orc.bf16_to_f32(kp).reshape(seq_len, D)
    vf = orc.bf16_to_f32(vp).reshape(seq_len, D)
    expected = np.empty((q_heads, D), dtype=np.float32)
    for h in range(q_heads):
        scores = (kf * qf[h][None, :]).astype(np.float32).sum(axis=1, dtype=np.float32) * scale
        wts = np.exp(scores - scores.max()).astype(np.float32)
        expected[h] = ((wts / wts.sum(dtype=np.float32))[:, None] * vf).sum(axis=0, dtype=np.float32)
    expected = orc.bf16_to_f32(orc.f32_to_bf16(expected))

    page = 16
    pages = -(-seq_len // page)
    cfg = (1, pages, page, pages, 1, 1, D, 0)
    cache_k = np.zeros(pages * page * D, dtype=np.uint16)
    cache_v = np.zeros_like(cache_k)
    cache_k[:seq_len * D] = kp.reshape(-1)
    cache_v[:seq_len * D] = vp.reshape(-1)
    table = np.arange(pages, dtype=np.int32).reshape(1, pages)
    seq = np.array([seq_len], dtype=np.int32)
    qrow = np.ascontiguousarray(qp[seq_len - 1:seq_len])
    out, *_ = orc.decode_attention_ref(qrow, cache_k, cache_v, table, seq, cfg, 0, float(scale), 20, 2, 1, q_heads)
    assert np.abs(orc.bf16_to_f32(out).reshape(q_heads, D) - expected).max() <= 0.03125
    out64, _ = orc.decode_attention_f64(qrow, cache_k, cache_v, table, seq, cfg, 0, float(scale), 1, q_heads)
    assert np.abs(out64.reshape(q_heads, D) - expected).max() <= 0.03125
