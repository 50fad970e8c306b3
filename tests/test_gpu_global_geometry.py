"""Decode attention for the reference's native global-layer geometry (16 query heads on one KV head of
512 dims, partial rotary 128, V derived from raw K; src/gemma4.h:19-21,28) through the C-ABI: the
tensor-core kernel against the double-precision oracle on the same bf16 cache (stated bf16 tolerance),
and one layer-step (append + attention) with cache bytes and prepared q bit-exact."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from tests import helpers
from tests.gpu_util import dev, host_u16, need_gpu
from tests.helpers import ATTN_MAX_ABS, ATTN_MAX_REL, LSE_MAX_ABS, attention_error, make_attn_case
from tests.test_gpu_decode_attention import DeviceCase, check

pytestmark = [pytest.mark.gpu, need_gpu]

GEOMETRY = dict(kv_heads=1, q_heads=16, head_dim=512)


@pytest.mark.parametrize("name,kw", [
    ("mixed_page16", dict(seq_lens=[300, 17, 1, 64, 129, 2047, 0, 8])),
    ("reference_bench_shape_page64", dict(seq_lens=[4096], page_size=64)),
    ("long_and_short", dict(seq_lens=[9000, 900, 33])),
    ("ring", dict(seq_lens=[5000, 90, 1024, 1025], window=1024)),
    ("outlier_keys", dict(seq_lens=[3000, 777], outlier_frac=0.01)),
    ("page8_unaligned_lengths", dict(seq_lens=[1001, 15, 16, 17], page_size=8)),
])
def test_gqa16_attention_against_double_precision(kv, orc, name, kw):
    case = make_attn_case(77, **GEOMETRY, **kw)
    d = DeviceCase(kv, case)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for num_splits in (kv.plan_balanced(case.batch, sms), 4):
        out, lse, _ = d.run(0, num_splits)
        check(orc, case, out, lse)


def test_gqa16_unmapped_pages_are_skipped(kv, orc):
    case = make_attn_case(78, seq_lens=[500, 260], **GEOMETRY)
    case.page_table[0, 3] = -1
    case.page_table[1, 0] = case.cfg[1] + 5          # outside the pool
    d = DeviceCase(kv, case)
    out, lse, _ = d.run(0, 40)
    check(orc, case, out, lse)


def test_gqa16_rejects_fixed_splits(kv):
    case = make_attn_case(79, seq_lens=[64], **GEOMETRY)
    d = DeviceCase(kv, case)
    B, H, D = 1, 16, 512
    out = torch.zeros((B, H, D), dtype=torch.int16, device="cuda")
    pm = torch.zeros(B * H * 4, dtype=torch.float32, device="cuda")
    pacc = torch.zeros(B * H * 4 * D, dtype=torch.float32, device="cuda")
    assert kv.decode_attention(out, None, d.q, d.ck, d.cv, d.cfg, d.table, d.seq, 0, case.scale, 64, 4, B, H,
                               pm, pm.clone(), pacc, None, check=False) == kv.CUDA_ERROR_INVALID_VALUE


def test_gqa16_layer_step_append_then_attend(kv, orc):
    """Three sequences, 9 decode steps through b200kv_decode_layer_step_bf16: rotary 128 of 512 dims,
    V = scale-free norm of raw K. Cache and prepared q bit-exact (IEEE mode), attention within tolerance."""
    rng = np.random.default_rng(5)
    H, HKV, D, ROT = 16, 1, 512, 128
    start = np.array([0, 37, 300], np.int32)
    steps = 9
    acase = helpers.make_append_case(9, start, kv_heads=HKV, q_heads=H, head_dim=D, rotary_dim=ROT, window=0,
                                     max_pos=int(start.max()) + steps + 1, has_v=False, theta=1.0e6)
    cfg_t = acase.cfg
    cfg = kv.make_kv_config(*cfg_t)
    elems = cfg_t[0] * cfg_t[1] * cfg_t[2] * cfg_t[5] * cfg_t[6]
    ck = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
    cv = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
    dck, dcv = dev(ck), dev(cv)
    B = start.size
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    num_splits = kv.plan_balanced(B, sms)
    dqp = torch.zeros((B, H, D), dtype=torch.int16, device="cuda")
    out = torch.zeros_like(dqp)
    lse = torch.zeros((B, H), dtype=torch.float32, device="cuda")
    pm = torch.zeros(B * H * num_splits, dtype=torch.float32, device="cuda"); pl = torch.zeros_like(pm)
    pacc = torch.zeros(B * H * num_splits * D, dtype=torch.float32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    table, qw, kw_, cos, sin = dev(acase.page_table), dev(acase.q_w), dev(acase.k_w), dev(acase.cos), dev(acase.sin)
    scale = 1.0 / np.sqrt(D)
    for t in range(steps):
        pos = (start + t).astype(np.int32)
        length = (pos + 1).astype(np.int32)
        q = helpers.bf16_normal(rng, (B, H, D))
        k = helpers.bf16_normal(rng, (B, HKV, D))
        dq, dk, dpos, dlen = dev(q), dev(k), dev(pos), dev(length)
        a = kv.LayerStepArgs()
        a.q, a.out, a.lse = dqp.data_ptr(), out.data_ptr(), lse.data_ptr()
        a.partial_m, a.partial_l, a.partial_acc = pm.data_ptr(), pl.data_ptr(), pacc.data_ptr()
        a.cache_k, a.cache_v, a.cache_config = dck.data_ptr(), dcv.data_ptr(), cfg
        a.page_table, a.token_position, a.seq_lengths = table.data_ptr(), dpos.data_ptr(), dlen.data_ptr()
        a.cache_layer, a.split_size, a.num_splits, a.softmax_scale = 0, 0, num_splits, scale
        a.raw_q, a.raw_k, a.raw_v = dq.data_ptr(), dk.data_ptr(), None
        a.q_norm_weight, a.k_norm_weight, a.cos, a.sin = qw.data_ptr(), kw_.data_ptr(), cos.data_ptr(), sin.data_ptr()
        a.batch_count, a.q_heads, a.rotary_dim, a.norm_mode = B, H, ROT, kv.NORM_IEEE
        a.status = status.data_ptr()
        kv.decode_layer_step(a)
        torch.cuda.synchronize()
        assert status[0].item() == 0
        qp = np.zeros((B, H, D), np.uint16)
        orc.decode_append(qp, ck, cv, cfg_t, acase.page_table, pos, 0, q, k, None, acase.q_w, acase.k_w,
                          acase.cos, acase.sin, B, H, ROT)
        assert np.array_equal(host_u16(dck), ck) and np.array_equal(host_u16(dcv), cv), t
        assert np.array_equal(host_u16(dqp), qp.reshape(-1)), t
        ref, ref_lse = orc.decode_attention_f64(qp, ck, cv, acase.page_table, length, cfg_t, 0, scale, B, H)
        max_abs, max_rel = attention_error(host_u16(out), ref)
        assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (t, max_abs, max_rel)
        assert np.abs(lse.cpu().numpy() - ref_lse).max() <= LSE_MAX_ABS
