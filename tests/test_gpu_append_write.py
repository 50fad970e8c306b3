"""GPU parity of the cache write, the fused decode append, the prompt prep and the runtime
state, through the C-ABI, against the CPU oracle. Cache bytes are compared bit for bit."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from tests import helpers
from tests.gpu_util import dev, host_u16, need_gpu, read_device
from tests.helpers import closed_form_value, make_append_case

pytestmark = [pytest.mark.gpu, need_gpu]


def test_invalid_page_write_is_a_noop(kv):
    """tests/test_kv_cache.cu:94-133 run against the product library."""
    cfg = kv.make_kv_config(1, 2, 4, 2, 1, 2, 16, 0)
    n = 2 * 16
    k = dev(closed_form_value(43000 + np.arange(n)))
    v = dev(closed_form_value(44000 + np.arange(n)))
    ck = torch.zeros(cfg.cache_elements(), dtype=torch.int16, device="cuda")
    cv = torch.zeros_like(ck)
    table = dev(np.full(2, -1, dtype=np.int32))
    kv.kv_cache_write(ck, cv, cfg, table, dev(np.array([1], np.int32)), dev(np.array([0], np.int32)), 1, 0, k, v)
    torch.cuda.synchronize()
    assert not ck.any() and not cv.any()


@pytest.mark.parametrize("window,page_size,heads,dim", [(0, 16, 8, 256), (1024, 16, 8, 256), (0, 64, 1, 512),
                                                        (8, 4, 2, 16), (0, 2, 3, 40)])
def test_cache_write_bit_exact(kv, orc, window, page_size, heads, dim):
    rng = np.random.default_rng(42)
    batch, layers = 3, 2
    mpps = 70 if window == 0 else max(1, -(-(window + page_size - 1) // page_size))
    tokens = 500
    table, num_pages = helpers.build_page_table(rng, batch, mpps, [mpps] * batch)
    table[1, 3 % mpps] = -1                     # an unmapped slot
    if mpps > 5:
        table[2, 5] = num_pages + 7             # outside the pool
    cfg = kv.make_kv_config(layers, num_pages, page_size, mpps, batch, heads, dim, window)
    tb = rng.integers(-1, batch + 1, size=tokens).astype(np.int32)      # includes -1 and batch (invalid)
    tp = rng.integers(-2, mpps * page_size + 3 * page_size, size=tokens).astype(np.int32)
    # distinct destinations: two valid tokens may hit the same row, the order of which the GPU does not
    # define; make (batch, position mod capacity) unique
    seen, keep = set(), []
    cap = mpps * page_size
    for i in range(tokens):
        key = (int(tb[i]), int(tp[i]) % cap if tp[i] >= 0 else -1 - i)
        if key not in seen:
            seen.add(key)
            keep.append(i)
    tb, tp = tb[keep], tp[keep]
    k = helpers.bf16_normal(rng, (tb.size, heads, dim))
    v = helpers.bf16_normal(rng, (tb.size, heads, dim))
    ck = rng.integers(0, 65536, size=cfg.cache_elements()).astype(np.uint16)
    cv = rng.integers(0, 65536, size=cfg.cache_elements()).astype(np.uint16)
    dck, dcv = dev(ck), dev(cv)
    kv.kv_cache_write(dck, dcv, cfg, dev(table), dev(tb), dev(tp), tb.size, 1, dev(k), dev(v))
    assert orc.kv_cache_write(ck, cv, cfg.astuple(), table, tb, tp, 1, k, v) == 0
    assert np.array_equal(host_u16(dck), ck)
    assert np.array_equal(host_u16(dcv), cv)


def _run_append(kv, case, norm_mode, cache_fill=0x7F7F):
    cfg = kv.make_kv_config(*case.cfg)
    elems = cfg.cache_elements()
    ck = np.full(elems, cache_fill, dtype=np.uint16)
    cv = np.full(elems, cache_fill ^ 0x1111, dtype=np.uint16)
    qp = np.full(case.q.shape, 0x5555, dtype=np.uint16)
    dck, dcv, dqp = dev(ck), dev(cv), dev(qp)
    kv.decode_append(dqp, dck, dcv, cfg, dev(case.page_table), dev(case.token_position), case.layer,
                     dev(case.q), dev(case.k), dev(case.v) if case.v is not None else None,
                     dev(case.q_w), dev(case.k_w), dev(case.cos), dev(case.sin),
                     case.token_position.size, case.q_heads, case.rotary_dim, norm_mode)
    return host_u16(dqp), host_u16(dck), host_u16(dcv), (qp, ck, cv)


APPEND_CASES = [
    dict(positions=[1024], window=1024, ring_pages=64, max_pos=1025),          # config 1: tight ring wraps
    dict(positions=[1040], window=1024, max_pos=1041),                          # slack ring (65 pages) wraps
    dict(positions=[0, 15, 16, 17, 4095], window=0, theta=1e6),                 # linear, theta 1e6
    dict(positions=[3, -1, 40], window=1024),                                   # negative position skipped
    dict(positions=[7, 300], window=0, kv_heads=1, q_heads=16, head_dim=512, rotary_dim=128,
         exponent_dim=512, theta=1e6, has_v=False),                             # reference-native global
    dict(positions=[5, 6, 7, 8], window=0, kv_heads=4, q_heads=8),              # a KV-head shard
]


@pytest.mark.parametrize("kw", APPEND_CASES)
def test_fused_append_bit_exact_ieee(kv, orc, kw):
    case = make_append_case(101, **kw)
    if len(kw["positions"]) > 2 and kw.get("kv_heads", 8) == 8 and kw["window"] == 0:
        case.page_table[2, 1] = -1      # position 16..31 of sequence 2 unmapped: K/V dropped, q still prepared
    got_q, got_k, got_v, (qp, ck, cv) = _run_append(kv, case, kv.NORM_IEEE)
    orc.decode_append(qp, ck, cv, case.cfg, case.page_table, case.token_position, case.layer, case.q, case.k,
                      case.v, case.q_w, case.k_w, case.cos, case.sin, case.token_position.size, case.q_heads,
                      case.rotary_dim)
    assert np.array_equal(got_k, ck)
    assert np.array_equal(got_v, cv)
    assert np.array_equal(got_q, qp.reshape(-1))


@pytest.mark.parametrize("kw", APPEND_CASES[:3])
def test_fused_append_rsqrt_mode_within_one_ulp(kv, orc, kw):
    """Default mode evaluates the norm scale with rsqrt.approx as the reference's GPU code does; against
    the IEEE host oracle it may differ by one bf16 step on a few elements and nowhere else."""
    case = make_append_case(102, **kw)
    got_q, got_k, got_v, (qp, ck, cv) = _run_append(kv, case, kv.NORM_RSQRT_APPROX)
    orc.decode_append(qp, ck, cv, case.cfg, case.page_table, case.token_position, case.layer, case.q, case.k,
                      case.v, case.q_w, case.k_w, case.cos, case.sin, case.token_position.size, case.q_heads,
                      case.rotary_dim)
    for got, want in ((got_k, ck), (got_v, cv), (got_q, qp.reshape(-1))):
        a = orc.bf16_to_f32(got).astype(np.float64)
        b = orc.bf16_to_f32(want).astype(np.float64)
        step = np.maximum(np.abs(b), 2.0 ** -100) * 2.0 ** -7
        assert np.all(np.abs(a - b) <= step)
        assert (got != want).mean() < 0.02


def test_append_round_trip_through_a_wrapping_ring(kv, orc):
    """Append positions 0..1100 one at a time into a tight 1024-token ring, then read the ring back:
    every slot holds the row of the newest position that maps to it (encode -> overwrite -> gather)."""
    rng = np.random.default_rng(9)
    steps, window, ps = 1101, 1024, 16
    case = make_append_case(9, [0], window=window, ring_pages=64, max_pos=steps)
    cfg = kv.make_kv_config(*case.cfg)
    dck = torch.zeros(cfg.cache_elements(), dtype=torch.int16, device="cuda")
    dcv = torch.zeros_like(dck)
    k_all = helpers.bf16_normal(rng, (steps, 8, 256))
    v_all = helpers.bf16_normal(rng, (steps, 8, 256))
    q = dev(case.q)
    dk_all, dv_all = dev(k_all), dev(v_all)
    dq_out = torch.zeros_like(q)
    table, qw, kw_, cos, sin = dev(case.page_table), dev(case.q_w), dev(case.k_w), dev(case.cos), dev(case.sin)
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    for t in range(steps):
        pos.fill_(t)
        kv.decode_append(dq_out, dck, dcv, cfg, table, pos, 0, q, dk_all[t], dv_all[t], qw, kw_, cos, sin,
                         1, 16, 256, kv.NORM_IEEE)
    got_k, got_v = host_u16(dck), host_u16(dcv)
    for t in range(steps - window, steps):          # the live window
        phys = int(case.page_table[0, (t // ps) % 64])
        base = orc.cache_offset(case.cfg, 0, phys, t % ps, 0, 0)
        for h in (0, 7):
            want_k = orc.prep_weighted_rope_head(k_all[t, h].copy(), case.k_w, case.cos[t].copy(), case.sin[t].copy(), 256)
            assert np.array_equal(got_k[base + h * 256: base + (h + 1) * 256], want_k)
            assert np.array_equal(got_v[base + h * 256: base + (h + 1) * 256], orc.prep_scale_free_head(v_all[t, h].copy()))


@pytest.mark.parametrize("geometry", [(16, 8, 256, 256, True), (16, 1, 512, 128, False)])
def test_prefill_prep_bit_exact_ieee(kv, orc, geometry):
    q_heads, kv_heads, D, rot, has_v = geometry
    rng = np.random.default_rng(77)
    rows = 65
    pos = rng.integers(0, 500, size=rows).astype(np.int32)
    pos[7] = -1                                         # skipped row keeps its old contents
    cos, sin = orc.fill_rope_tables(500, rot // 2, 10000.0 if has_v else 1e6, D)
    q = helpers.bf16_normal(rng, (rows, q_heads, D))
    k = helpers.bf16_normal(rng, (rows, kv_heads, D))
    v = helpers.bf16_normal(rng, (rows, kv_heads, D)) if has_v else None
    qw = helpers.bf16_normal(rng, (D,), 0.05, 1.0)
    kw_ = helpers.bf16_normal(rng, (D,), 0.05, 1.0)
    dq, dk, dv = (torch.zeros(x.shape, dtype=torch.int16, device="cuda") for x in (q, k, k))
    kv.prefill_prep(dq, dk, dv, dev(q), dev(k), dev(v) if has_v else None, dev(qw), dev(kw_), dev(cos), dev(sin),
                    dev(pos), rows, q_heads, kv_heads, D, rot, kv.NORM_IEEE)
    wq, wk, wv = orc.prefill_prep(q, k, v, qw, kw_, cos, sin, pos, q_heads, kv_heads, D, rot)
    assert np.array_equal(host_u16(dq), wq.reshape(-1))
    assert np.array_equal(host_u16(dk), wk.reshape(-1))
    assert np.array_equal(host_u16(dv), wv.reshape(-1))


def test_global_prep_pins_of_the_reference_test(kv, orc):
    """tests/test_flash_attention.cu:232-325 against the product kernel (default rsqrt mode): K-derived
    scale-free V within 2^-8, RoPE at the absolute positions {2, 4} within 2^-8."""
    D, half, rows = 512, 64, 2
    k = closed_form_value(110000 + np.arange(rows * D)).reshape(rows, 1, D)
    q = np.zeros((rows, 16, D), dtype=np.uint16)
    w = orc.f32_to_bf16(np.ones(D, dtype=np.float32))
    pos = np.array([2, 4], dtype=np.int32)
    cos = np.ones((5, half), dtype=np.float32); sin = np.zeros((5, half), dtype=np.float32)
    cos[2, 0], sin[2, 0], cos[4, 0], sin[4, 0] = 0.0, 1.0, 0.0, -1.0
    dq = torch.zeros(q.shape, dtype=torch.int16, device="cuda")
    dk = torch.zeros(k.shape, dtype=torch.int16, device="cuda"); dv = torch.zeros_like(dk)
    kv.prefill_prep(dq, dk, dv, dev(q), dev(k), None, dev(w), dev(w), dev(cos), dev(sin), dev(pos),
                    rows, 16, 1, D, 128)
    kf = orc.bf16_to_f32(k).reshape(rows, D)
    inv = (1.0 / np.sqrt((kf.astype(np.float64) ** 2).mean(axis=1) + 1e-6)).astype(np.float32)
    got_v = orc.bf16_to_f32(host_u16(dv)).reshape(rows, D)
    assert np.abs(got_v - orc.bf16_to_f32(orc.f32_to_bf16(kf * inv[:, None]))).max() <= 0.00390625
    got_k = orc.bf16_to_f32(host_u16(dk)).reshape(rows, D)
    for r in range(rows):
        c, s = cos[pos[r], 0], sin[pos[r], 0]
        lo, hi = kf[r, 0] * inv[r], kf[r, half] * inv[r]
        assert abs(got_k[r, 0] - (lo * c - hi * s)) <= 0.00390625 + 2.0 ** -8 * abs(lo * c - hi * s)
        assert abs(got_k[r, half] - (lo * s + hi * c)) <= 0.00390625 + 2.0 ** -8 * abs(lo * s + hi * c)
    assert not host_u16(dq).any()          # q = 0 stays 0


def test_runtime_state_metadata_on_device(kv):
    """tests/test_runtime_state.cu:29-140 through the C handle: device copies of the metadata after
    prefill(64) and one decode step, the all-or-nothing failing step, and the RoPE tables."""
    rt = kv.RuntimeState(2, 66, 64)
    rt.prepare_prefill(64)
    torch.cuda.synchronize()
    v = rt.view()

    def d_i32(ptr, n):
        return read_device(ptr, n, np.int32)

    assert v.token_count == 128
    assert list(d_i32(v.seq_lengths, 2)) == [64, 64]
    tb, tp = d_i32(v.token_batch, 128), d_i32(v.token_position, 128)
    assert (tb[63], tp[63], tb[64], tp[64]) == (0, 63, 1, 0)
    assert rt.host_array("h_sliding_page_table")[0] >= 0
    assert rt.host_array("h_sliding_page_table")[v.sliding_cache_config.max_pages_per_seq] >= 0
    assert rt.host_array("h_global_page_table")[0] >= 0
    assert rt.host_array("h_global_page_table")[v.global_cache_config.max_pages_per_seq] >= 0

    rt.prepare_decode_step()
    torch.cuda.synchronize()
    v = rt.view()
    assert v.token_count == 2
    assert list(d_i32(v.seq_lengths, 2)) == [65, 65]
    assert list(d_i32(v.token_batch, 2)) == [0, 1] and list(d_i32(v.token_position, 2)) == [64, 64]
    assert d_i32(v.sliding_page_table, 4)[1] == 1 and d_i32(v.global_page_table, 4)[1] == 1

    rt.host_array("h_seq_lengths")[:] = [64, 66]
    names = ["h_seq_lengths", "h_token_batch", "h_token_position", "h_sliding_page_table", "h_global_page_table",
             "h_sliding_slot_logical_pages", "h_global_slot_logical_pages"]
    before = {n: rt.host_array(n).copy() for n in names}
    assert rt.prepare_decode_step(check=False) == kv.CUDA_ERROR_INVALID_VALUE
    for n in names:
        assert np.array_equal(rt.host_array(n), before[n]), n
    rt.close()

    rt = kv.RuntimeState(1, 4, 4)
    torch.cuda.synchronize()
    v = rt.view()

    def d_f32(ptr, n):
        return read_device(ptr, n, np.float32)

    import math
    sc, ss, gc = d_f32(v.sliding_cos, 4 * 128), d_f32(v.sliding_sin, 4 * 128), d_f32(v.global_cos, 4 * 64)
    assert abs(sc[128] - math.cos(1.0)) <= 1e-6 and abs(ss[128] - math.sin(1.0)) <= 1e-6
    assert abs(gc[64 + 1] - math.cos(1e6 ** (-2.0 / 512.0))) <= 1e-6
    assert v.sliding_cache_config.astuple() == (40, 1, 4, 1, 1, 8, 256, 4)
    assert v.global_cache_config.astuple() == (8, 1, 4, 1, 1, 1, 512, 0)
    rt.close()
    assert kv.RuntimeState(0, 4, 4, check=False).status == kv.CUDA_ERROR_INVALID_VALUE


@pytest.mark.parametrize("window,seq_len", [(64, 200), (64, 64), (64, 17), (0, 200)])
def test_prompt_cache_fill_keeps_the_live_tail(kv, orc, window, seq_len):
    """b200kv_prefill_cache_fill_bf16 against the reference's write step
    (src/gemma4_prefill_megakernel.cu:189-207) restated with the oracle's cache write: every row for a
    linear cache or a prompt within the window, else one write of the last `window` rows per sequence."""
    rng = np.random.default_rng(77)
    batch, page_size, heads, dim = 3, 16, 8, 256
    mpps = -(-seq_len // page_size) if window == 0 else -(-(window + page_size - 1) // page_size)
    table, num_pages = helpers.build_page_table(rng, batch, mpps, [mpps] * batch)
    cfg = kv.make_kv_config(2, num_pages, page_size, mpps, batch, heads, dim, window)
    rows = batch * seq_len
    tb = np.repeat(np.arange(batch, dtype=np.int32), seq_len)           # gemma4_runtime_prepare_prefill's layout
    tp = np.tile(np.arange(seq_len, dtype=np.int32), batch)
    k = helpers.bf16_normal(rng, (rows, heads, dim))
    v = helpers.bf16_normal(rng, (rows, heads, dim))
    ck = rng.integers(0, 65536, size=cfg.cache_elements()).astype(np.uint16)
    cv = rng.integers(0, 65536, size=cfg.cache_elements()).astype(np.uint16)
    dck, dcv = dev(ck), dev(cv)
    kv.prefill_cache_fill(dck, dcv, cfg, dev(table), dev(tb), dev(tp), batch, seq_len, 1, dev(k), dev(v))
    if window == 0 or seq_len <= window:
        assert orc.kv_cache_write(ck, cv, cfg.astuple(), table, tb, tp, 1, k, v) == 0
    else:
        for b in range(batch):
            lo = b * seq_len + seq_len - window
            sl = slice(lo, lo + window)
            assert orc.kv_cache_write(ck, cv, cfg.astuple(), table, np.ascontiguousarray(tb[sl]),
                                      np.ascontiguousarray(tp[sl]), 1, np.ascontiguousarray(k[sl]),
                                      np.ascontiguousarray(v[sl])) == 0
    torch.cuda.synchronize()
    assert np.array_equal(host_u16(dck), ck) and np.array_equal(host_u16(dcv), cv)
    assert kv.prefill_cache_fill(dck, dcv, cfg, dev(table), dev(tb), dev(tp), -1, seq_len, 1, dev(k), dev(v),
                                 check=False) == kv.CUDA_ERROR_INVALID_VALUE
    assert kv.prefill_cache_fill(dck, dcv, cfg, dev(table), dev(tb), dev(tp), batch, seq_len, 2, dev(k), dev(v),
                                 check=False) == kv.CUDA_ERROR_INVALID_VALUE
