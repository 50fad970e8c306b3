"""The allocation-free decode entry point (b200kv_decode_attention_static_scratch_bf16).

Some callers of this library cannot provide the split-partial scratch that the regular decode call
wants: an engine that committed all device memory to its page pool, a plug-in without an allocator, a
latency path that must avoid cudaMalloc's device-wide synchronisation. For them the library carries a
fixed 16 MiB array on the device. This test calls that entry point through the C-ABI twice in a row
(the second call sees the first call's leftovers in the shared array) and requires the same result as
the regular entry point with caller-owned scratch, within the decode tolerance of the other GPU tests.
It is collected last so that a run that stops at the first failure has already run everything else.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from tests.gpu_util import dev, host_u16, need_gpu
from tests.helpers import ATTN_MAX_ABS, ATTN_MAX_REL, LSE_MAX_ABS, attention_error, make_attn_case

pytestmark = [pytest.mark.gpu, need_gpu]


def _run_both(kv, orc, case, split_size, num_splits):
    cfg = kv.make_kv_config(*case.cfg)
    B, H, D = case.batch, case.q_heads, case.head_dim
    q, ck, cv = dev(case.q), dev(case.cache_k), dev(case.cache_v)
    table, seq = dev(case.page_table), dev(case.seq_lengths)

    def buffers():
        return (torch.full((B, H, D), 0x7FC0, dtype=torch.int16, device="cuda"),
                torch.full((B, H), float("nan"), dtype=torch.float32, device="cuda"),
                torch.zeros(4, dtype=torch.int32, device="cuda"))

    out_a, lse_a, st_a = buffers()
    rows = B * H * num_splits
    pm = torch.full((rows,), float("nan"), dtype=torch.float32, device="cuda")
    pl = torch.full_like(pm, float("nan"))
    pacc = torch.full((rows * D,), float("nan"), dtype=torch.float32, device="cuda")
    kv.decode_attention(out_a, lse_a, q, ck, cv, cfg, table, seq, case.layer, case.scale, split_size, num_splits,
                        B, H, pm, pl, pacc, st_a)
    out_b, lse_b, st_b = buffers()
    kv.decode_attention_static_scratch(out_b, lse_b, q, ck, cv, cfg, table, seq, case.layer, case.scale,
                                       split_size, num_splits, B, H, st_b)
    torch.cuda.synchronize()
    assert st_a[0].item() == 0 and st_b[0].item() == 0
    a, b = host_u16(out_a).reshape(B, H, D), host_u16(out_b).reshape(B, H, D)
    # same kernels, same inputs: against each other within the decode tolerance, and each against the oracle
    max_abs, max_rel = attention_error(b, orc.bf16_to_f32(a))
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL
    la, lb = lse_a.cpu().numpy(), lse_b.cpu().numpy()
    finite = np.isfinite(la)
    assert np.array_equal(np.isfinite(lb), finite)
    assert np.abs(la[finite] - lb[finite]).max(initial=0.0) <= LSE_MAX_ABS
    ref, _ = orc.decode_attention_f64(case.q, case.cache_k, case.cache_v, case.page_table, case.seq_lengths,
                                      case.cfg, case.layer, case.scale, B, H)
    max_abs, max_rel = attention_error(b, ref)
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL


def test_static_scratch_matches_caller_scratch_on_two_calls_in_a_row(kv, orc):
    first = make_attn_case(501, [2000, 700, 64], window=0)
    _run_both(kv, orc, first, 64, 32)                 # fills a large part of the shared array
    second = make_attn_case(502, [300, 1025], window=1024)
    _run_both(kv, orc, second, 40, 30)                # fewer live splits: leftovers of call one stay around them
    third = make_attn_case(503, [90], window=0)
    _run_both(kv, orc, third, 128, 1)                 # single split: no scratch at all


def test_static_scratch_on_the_balanced_partition_and_the_wide_head_geometry(kv, orc):
    """The library's default partition (split_size 0: key ranges balanced over a fixed grid, one scratch slot
    per CTA and sequence boundary) and the 16-query-heads-on-one-KV-head-of-512 geometry through the shared
    array, each twice in a row and interleaved, against the caller-scratch entry point and the oracle. With
    split_size 0 a single split is refused: that partition always needs its scratch."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    ragged = make_attn_case(505, [3000, 17, 1500, 260], window=0)
    wide = make_attn_case(506, [2100, 40], window=0, kv_heads=1, q_heads=16, head_dim=512)
    ring = make_attn_case(507, [1500], window=1024)
    for case in (ragged, wide, ragged, wide, ring, ring):
        _run_both(kv, orc, case, 0, kv.plan_balanced(case.batch, sms))
    cfg = kv.make_kv_config(*ring.cfg)
    out = torch.zeros((1, 16, 256), dtype=torch.int16, device="cuda")
    code = kv.decode_attention_static_scratch(out, None, dev(ring.q), dev(ring.cache_k), dev(ring.cache_v), cfg,
                                              dev(ring.page_table), dev(ring.seq_lengths), 0, ring.scale, 0, 1, 1, 16,
                                              check=False)
    assert code == kv.CUDA_ERROR_INVALID_VALUE


def test_static_scratch_refuses_what_does_not_fit(kv, capfd):
    case = make_attn_case(504, [64], window=0)
    cfg = kv.make_kv_config(*case.cfg)
    out = torch.zeros((1, 16, 256), dtype=torch.int16, device="cuda")
    q, ck, cv = dev(case.q), dev(case.cache_k), dev(case.cache_v)
    table, seq = dev(case.page_table), dev(case.seq_lengths)
    rows_that_fit = kv.STATIC_SCRATCH_BYTES // 4 // (256 + 2)
    too_many_splits = rows_that_fit // 16 + 8
    code = kv.decode_attention_static_scratch(out, None, q, ck, cv, cfg, table, seq, 0, case.scale, 8,
                                              too_many_splits, 1, 16, check=False)
    assert code == kv.CUDA_ERROR_INVALID_VALUE
    assert "built-in scratch" in capfd.readouterr().err
    torch.cuda.synchronize()
    assert not out.any()                               # nothing was launched
