"""FP8 e4m3 KV cache (one fp32 scale per 16-token page and KV head): quantise-on-append and fused
dequant in decode attention, through the C-ABI, against the CPU oracle.

Stored bytes and scales: bit-exact against the oracle's statement of the rule. Attention on the same
quantised cache: the bf16 decode tolerance (2^-6). Attention against the bf16-cache result on the same
inputs: max_abs <= 0.05 and mean_abs <= 5e-3 (the quantisation itself; stated FP8 tolerance).
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from tests import helpers
from tests.gpu_util import dev, host_u16, host_u8, need_gpu
from tests.helpers import ATTN_MAX_ABS, ATTN_MAX_REL, LSE_MAX_ABS, attention_error

pytestmark = [pytest.mark.gpu, need_gpu]

FP8_MAX_ABS = 0.05
FP8_MEAN_ABS = 5.0e-3
H, HQ, D, PAGE = 8, 16, 256, 16


def _cache(cfg):
    elems = cfg[0] * cfg[1] * cfg[2] * cfg[5] * cfg[6]
    scales = cfg[0] * cfg[1] * cfg[5]
    return (np.zeros(elems, np.uint8), np.zeros(elems, np.uint8), np.zeros(scales, np.float32),
            np.zeros(scales, np.float32))


def test_fused_append_fp8_bit_exact_over_many_steps(kv, orc):
    """Two sequences, 45 decode steps each, a tight 32-token ring for good measure: every step the
    fused kernel preps and quantises one row per sequence; bytes and scales must equal the oracle's."""
    rng = np.random.default_rng(321)
    steps, window, pages = 45, 32, 2
    case = helpers.make_append_case(5, [0, 0], window=window, ring_pages=pages, max_pos=steps + 3)
    cfg = kv.make_kv_config(*case.cfg)
    ck, cv, sk, sv = _cache(case.cfg)
    dck, dcv, dsk, dsv = dev(ck), dev(cv), dev(sk), dev(sv)
    table, qw, kw_, cos, sin = dev(case.page_table), dev(case.q_w), dev(case.k_w), dev(case.cos), dev(case.sin)
    dq = torch.zeros((2, HQ, D), dtype=torch.int16, device="cuda")
    batch_ids = np.array([0, 1], np.int32)
    one = np.array([1, 1], np.int32)
    for t in range(steps):
        pos = np.array([t, t + 2], np.int32)
        q = helpers.bf16_normal(rng, (2, HQ, D))
        k = helpers.bf16_normal(rng, (2, H, D), std=float(rng.choice([0.3, 1.0, 5.0])))   # scale jumps
        v = helpers.bf16_normal(rng, (2, H, D), std=float(rng.choice([0.3, 1.0, 5.0])))
        kv.decode_append_fp8(dq, dck, dcv, dsk, dsv, cfg, table, dev(pos), 0, dev(q), dev(k), dev(v), qw, kw_,
                             cos, sin, 2, HQ, D, kv.NORM_IEEE)
        qp, kp, vp = orc.prefill_prep(q, k, v, case.q_w, case.k_w, case.cos, case.sin, pos, HQ, H, D, D)
        orc.fp8_append(ck, cv, sk, sv, case.cfg, case.page_table, batch_ids, pos, one, 0, kp, vp)
        if t % 9 == 0 or t == steps - 1:
            torch.cuda.synchronize()
            assert np.array_equal(host_u16(dq), qp.reshape(-1))
            assert np.array_equal(host_u8(dck), ck), t
            assert np.array_equal(host_u8(dcv), cv), t
            assert np.array_equal(dsk.cpu().numpy(), sk) and np.array_equal(dsv.cpu().numpy(), sv)
    assert sk.min() > 0


def test_bulk_append_fp8_bit_exact(kv, orc):
    """Prompt-sized runs that start and end inside pages, one dropped run (batch out of range), one
    unmapped page; then a second call that continues two of the sequences mid-page."""
    rng = np.random.default_rng(654)
    batch, mpps = 4, 6
    table, num_pages = helpers.build_page_table(rng, batch, mpps, [mpps] * batch)
    table[2, 1] = -1
    cfg_t = (2, num_pages, PAGE, mpps, batch, H, D, 0)
    cfg = kv.make_kv_config(*cfg_t)
    ck, cv, sk, sv = _cache(cfg_t)
    dck, dcv, dsk, dsv = dev(ck), dev(cv), dev(sk), dev(sv)
    calls = [
        (np.array([0, 1, 2, 7, 3], np.int32), np.array([0, 5, 3, 0, 16], np.int32), np.array([37, 60, 40, 9, 1], np.int32)),
        (np.array([0, 3], np.int32), np.array([37, 17], np.int32), np.array([20, 50], np.int32)),
    ]
    for seq_batch, first, count in calls:
        rows = int(count.sum())
        start = np.concatenate([[0], np.cumsum(count)[:-1]]).astype(np.int32)
        k = helpers.bf16_normal(rng, (rows, H, D), std=2.0)
        v = helpers.bf16_normal(rng, (rows, H, D), std=0.5)
        kv.fp8_append_rows(dck, dcv, dsk, dsv, cfg, dev(table), dev(seq_batch), dev(first), dev(count), dev(start),
                           seq_batch.size, int(count.max()), 1, dev(k), dev(v))
        orc.fp8_append(ck, cv, sk, sv, cfg_t, table, seq_batch, first, count, 1, k, v)
        torch.cuda.synchronize()
        assert np.array_equal(host_u8(dck), ck) and np.array_equal(host_u8(dcv), cv)
        assert np.array_equal(dsk.cpu().numpy(), sk) and np.array_equal(dsv.cpu().numpy(), sv)
    assert ck.any() and not ck[: ck.size // 2].any()          # layer 0 untouched


def _quantised_case(kv, orc, seed, seq_lens, window=0, ring_pages=None):
    """A bf16 attention case and its fp8 twin: the cache rows of every live position are pushed through
    the bulk append (on the device), so the fp8 cache holds exactly what appending them would give."""
    case = helpers.make_attn_case(seed, seq_lens, window=window, ring_pages=ring_pages)
    cfg = kv.make_kv_config(*case.cfg)
    ps, mpps = case.cfg[2], case.cfg[3]
    ck8, cv8, sk, sv = _cache(case.cfg)
    d = dict(ck=dev(ck8), cv=dev(cv8), sk=dev(sk), sv=dev(sv))
    kf = case.cache_k.reshape(-1, ps, H, D)
    vf = case.cache_v.reshape(-1, ps, H, D)
    table = dev(case.page_table)
    for b, n in enumerate(case.seq_lengths):
        n = int(n)
        first = max(0, n - window) if window > 0 else 0
        if n - first <= 0:
            continue
        pos = np.arange(first, n)
        phys = case.page_table[b, (pos // ps) % mpps]
        rows_k = np.ascontiguousarray(kf[phys, pos % ps])          # [rows, H, D] in position order
        rows_v = np.ascontiguousarray(vf[phys, pos % ps])
        one = lambda x: dev(np.array([x], np.int32))
        kv.fp8_append_rows(d["ck"], d["cv"], d["sk"], d["sv"], cfg, table, one(b), one(first), one(n - first),
                           one(0), 1, n - first, 0, dev(rows_k), dev(rows_v))
        orc.fp8_append(ck8, cv8, sk, sv, case.cfg, case.page_table, np.array([b], np.int32),
                       np.array([first], np.int32), np.array([n - first], np.int32), 0, rows_k, rows_v)
    torch.cuda.synchronize()
    assert np.array_equal(host_u8(d["ck"]), ck8) and np.array_equal(d["sk"].cpu().numpy(), sk)
    return case, cfg, d, (ck8, cv8, sk, sv)


@pytest.mark.parametrize("name,kw", [
    ("mixed", dict(seq_lens=[300, 17, 1, 64, 129, 2047, 0, 8])),
    ("long", dict(seq_lens=[6000, 900])),
    ("ring", dict(seq_lens=[5000, 90, 1024, 1025], window=1024)),
])
def test_fp8_decode_attention(kv, orc, name, kw):
    case, cfg, d, (ck8, cv8, sk, sv) = _quantised_case(kv, orc, 4242, **kw)
    B = case.batch
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    q, table, seq = dev(case.q), dev(case.page_table), dev(case.seq_lengths)
    for num_splits in (kv.plan_balanced(B, sms), 3):
        rows = B * HQ * num_splits
        out = torch.full((B, HQ, D), 0x7FC0, dtype=torch.int16, device="cuda")
        lse = torch.full((B, HQ), float("nan"), dtype=torch.float32, device="cuda")
        pm = torch.full((rows,), float("nan"), dtype=torch.float32, device="cuda"); pl = pm.clone()
        pacc = torch.full((rows * D,), float("nan"), dtype=torch.float32, device="cuda")
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        kv.decode_attention_fp8(out, lse, q, d["ck"], d["cv"], d["sk"], d["sv"], cfg, table, seq, 0, case.scale,
                                num_splits, B, HQ, pm, pl, pacc, status)
        torch.cuda.synchronize()
        assert status[0].item() == 0
        got = host_u16(out).reshape(B, HQ, D)
        # same quantised cache, double precision: the kernel's own arithmetic error
        ref8, lse8 = orc.fp8_decode_attention_f64(case.q, ck8, cv8, sk, sv, case.page_table, case.seq_lengths,
                                                  case.cfg, 0, case.scale, B, HQ)
        max_abs, max_rel = attention_error(got, ref8)
        assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (max_abs, max_rel)
        fin = np.isfinite(lse8)
        got_lse = lse.cpu().numpy()
        assert np.array_equal(np.isneginf(got_lse), np.isneginf(lse8))
        assert np.abs(got_lse[fin] - lse8[fin]).max(initial=0.0) <= LSE_MAX_ABS
        # against the bf16 cache: the cost of quantising K and V to e4m3
        ref16, _ = orc.decode_attention_f64(case.q, case.cache_k, case.cache_v, case.page_table, case.seq_lengths,
                                            case.cfg, 0, case.scale, B, HQ)
        diff = np.abs(orc.bf16_to_f32(got).astype(np.float64) - ref16.reshape(B, HQ, D))
        w = case.cfg[7]
        for b, n in enumerate(case.seq_lengths):
            live = min(int(n), w) if w > 0 else int(n)
            if live >= 512:          # the stated band, quoted for contexts of hundreds of keys and more
                assert diff[b].max() <= FP8_MAX_ABS, (b, diff[b].max())
                assert diff[b].mean() <= FP8_MEAN_ABS, (b, diff[b].mean())
            elif live > 0:           # a handful of keys: bounded by one e4m3 step of the largest V value
                vmax = float(np.abs(orc.bf16_to_f32(case.cache_v)).max())
                assert diff[b].max() <= vmax * 2.0 ** -4 + 2.0 ** -6, (b, diff[b].max())


def test_fp8_rejects_what_it_is_not_built_for(kv):
    cfg4 = kv.make_kv_config(1, 4, 16, 4, 1, 4, 256, 0)
    assert kv.decode_attention_fp8(16, None, 16, 16, 16, 16, 16, cfg4, 16, 16, 0, 0.0625, 8, 1, 8, 16, 16, 16,
                                   stream=0, check=False) == kv.CUDA_ERROR_INVALID_VALUE
    cfg = kv.make_kv_config(1, 4, 16, 4, 1, 8, 256, 0)
    assert kv.decode_attention_fp8(16, None, 16, 16, 16, None, 16, cfg, 16, 16, 0, 0.0625, 8, 1, 16, 16, 16, 16,
                                   stream=0, check=False) == kv.CUDA_ERROR_INVALID_VALUE
    assert kv.fp8_append_rows(16, 16, 16, 16, cfg, 16, 16, 16, 16, 16, 0, 5, 0, 16, 16, stream=0, check=False) == 0
    assert kv.fp8_append_rows(16, 16, 16, 16, cfg, 16, 16, 16, 16, 16, 1, 5, 3, 16, 16, stream=0,
                              check=False) == kv.CUDA_ERROR_INVALID_VALUE
