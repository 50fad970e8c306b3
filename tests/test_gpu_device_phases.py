"""The device-side form of the path (include/gemma4_b200kv_device.cuh): append_phase, split_phase and reduce_phase
called from a cooperative kernel with grid-wide barriers in between, the way the reference's decode megakernel
calls its own phases (tests/cpp/device_phases_harness.cu; the library is not linked into that harness).
Checked against the library's append through the C ABI on a second copy of the state -- prepared q and cache
bytes must be the same bits, both being the reference GPU code's arithmetic -- and against the double-precision
oracle for the attention rows and the log-sum-exp.

Covers: a ring that wrapped, a ragged linear batch, split sizes 20 (the reference's), 64, one split (rows written
by the split phase itself), more splits than a sequence needs, an unmapped page, a sequence that is not appended,
V derived from raw K."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from tests import helpers
from tests.gpu_util import build_device_phases_harness, dev, host_u16, need_gpu
from tests.helpers import ATTN_MAX_ABS, ATTN_MAX_REL, LSE_MAX_ABS, attention_error

pytestmark = [pytest.mark.gpu, need_gpu]

HQ, H, D = 16, 8, 256


@pytest.fixture(scope="module")
def harness(kv):
    lib = ctypes.CDLL(str(build_device_phases_harness()))
    P, I, F = ctypes.c_void_p, ctypes.c_int32, ctypes.c_float
    lib.device_phases_layer_step.restype = ctypes.c_int
    lib.device_phases_layer_step.argtypes = [P, P, P, P, P, P, P, P, kv.KvConfig, P, P, P, P, P, P, P, P, P, P,
                                             I, I, I, I, I, F]
    return lib


@pytest.mark.parametrize("name,window,ring_pages,start,split_size,extra_splits,has_v,unmapped", [
    ("ring that wrapped, split 20", 64, 5, [100, 7, 64, 200], 20, 0, True, None),
    ("tight ring, split 64", 64, 4, [130, 64], 64, 0, True, None),
    ("ragged linear batch, split 20", 0, None, [300, 17, 0, 129, 2047], 20, 0, True, None),
    ("linear, more splits than needed", 0, None, [300, 17, 63], 37, 5, True, None),
    ("one split: rows from the split phase", 0, None, [90, 5], 128, 0, True, None),
    ("one split, ring", 64, 5, [100, 70], 64, 0, True, None),
    ("unmapped page, a sequence not appended, V from raw K", 0, None, [100, -1, 40], 16, 0, False, (0, 2)),
])
def test_device_phases_layer_step(kv, orc, harness, name, window, ring_pages, start, split_size, extra_splits, has_v,
                                  unmapped):
    rng = np.random.default_rng(23)
    start = np.asarray(start, np.int32)
    B = start.size
    acase = helpers.make_append_case(9, np.maximum(start, 0), window=window, ring_pages=ring_pages,
                                     max_pos=int(start.max()) + 2, has_v=has_v)
    if unmapped is not None:
        acase.page_table[unmapped] = -1
    cfg_t = acase.cfg
    cfg = kv.make_kv_config(*cfg_t)
    elems = cfg_t[0] * cfg_t[1] * cfg_t[2] * cfg_t[5] * cfg_t[6]
    ck = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
    cv = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
    pos = start.copy()
    length = np.where(start >= 0, start + 1, 9).astype(np.int32)
    live = [min(int(n), window) if window else int(n) for n in length]
    num_splits = max(1, -(-max(live) // split_size)) + extra_splits
    q = helpers.bf16_normal(rng, (B, HQ, D))
    k = helpers.bf16_normal(rng, (B, H, D))
    v = helpers.bf16_normal(rng, (B, H, D)) if has_v else None
    dq, dk, dv = dev(q), dev(k), (dev(v) if has_v else None)
    table, qw, kw_, cos, sin = (dev(x) for x in (acase.page_table, acase.q_w, acase.k_w, acase.cos, acase.sin))
    dpos, dlen = dev(pos), dev(length)
    scale = 1.0 / 16.0

    # the phases, from the cooperative harness
    ck1, cv1 = dev(ck), dev(cv)
    q1 = torch.full((B, HQ, D), 0x1234, dtype=torch.int16, device="cuda")
    out1 = torch.full((B, HQ, D), 0x7FC0, dtype=torch.int16, device="cuda")
    lse1 = torch.full((B, HQ), float("nan"), dtype=torch.float32, device="cuda")
    rows = B * HQ * num_splits
    pm = torch.full((rows,), float("nan"), dtype=torch.float32, device="cuda")
    pl, pacc = pm.clone(), torch.full((rows * D,), float("nan"), dtype=torch.float32, device="cuda")
    rc = harness.device_phases_layer_step(
        q1.data_ptr(), ck1.data_ptr(), cv1.data_ptr(), out1.data_ptr(), lse1.data_ptr(), pm.data_ptr(),
        pl.data_ptr(), pacc.data_ptr(), cfg, table.data_ptr(), dpos.data_ptr(), dlen.data_ptr(), dq.data_ptr(),
        dk.data_ptr(), dv.data_ptr() if has_v else None, qw.data_ptr(), kw_.data_ptr(), cos.data_ptr(),
        sin.data_ptr(), 0, split_size, num_splits, B, HQ, scale)
    assert rc == 0, (name, rc)

    # the library's append on a second copy: the same bits
    ck2, cv2 = dev(ck), dev(cv)
    q2 = torch.full((B, HQ, D), 0x1234, dtype=torch.int16, device="cuda")
    kv.decode_append(q2, ck2, cv2, cfg, table, dpos, 0, dq, dk, dv, qw, kw_, cos, sin, B, HQ, D,
                     kv.NORM_RSQRT_APPROX)
    torch.cuda.synchronize()
    assert torch.equal(q1, q2), name
    assert torch.equal(ck1, ck2) and torch.equal(cv1, cv2), name

    # attention rows and log-sum-exp against double precision over the cache as it is now
    ref, ref_lse = orc.decode_attention_f64(host_u16(q1).reshape(B, HQ, D), host_u16(ck1), host_u16(cv1),
                                            acase.page_table, length, cfg_t, 0, scale, B, HQ)
    got = host_u16(out1).reshape(B, HQ, D)
    assert not np.isnan(orc.bf16_to_f32(got)).any(), name
    max_abs, max_rel = attention_error(got, ref)
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (name, max_abs, max_rel)
    lse = lse1.cpu().numpy()
    finite = np.isfinite(ref_lse)
    assert np.array_equal(np.isneginf(lse), np.isneginf(ref_lse)), name
    assert np.abs(lse[finite] - ref_lse[finite]).max(initial=0.0) <= LSE_MAX_ABS, name
    if num_splits > 1:          # splits beyond a sequence's live keys never touch the scratch
        m = pm.cpu().numpy().reshape(B, HQ, num_splits)
        for b, n in enumerate(live):
            actual = -(-n // split_size)
            assert not np.isnan(m[b, :, :actual]).any() and np.isnan(m[b, :, actual:]).all(), (name, b)
