"""The one-launch layer-step (append fused into the balanced decode kernel) through
b200kv_decode_layer_step_bf16, against (a) the two-launch form on a second copy of the same state --
caches, prepared q, attention rows and LSE must be the same bits -- and (b) the CPU oracle: cache bytes
and prepared q exact, attention within the stated bf16 tolerance. A third copy of the state runs the same
steps through b200kv_decode_layer_step_tiled_bf16 (a CTA per sequence, KV head and key range; partials
merged by the last CTA through tickets): caches and prepared q the same bits again, attention rows within
the tolerance (another summation order), tickets back at zero after every step.

Covers: sliding ring that wraps every few steps, linear cache, ragged batch, a sequence that is not
appended (position -1), an unmapped page, lengths that do not contain the new position (the row is
still appended), both norm modes, V derived from raw K."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from tests import helpers
from tests.gpu_util import dev, host_u16, need_gpu
from tests.helpers import ATTN_MAX_ABS, ATTN_MAX_REL, LSE_MAX_ABS, attention_error

pytestmark = [pytest.mark.gpu, need_gpu]

HQ, H, D = 16, 8, 256


class _State:
    """Device copy of everything one layer-step touches."""

    def __init__(self, kv, acase, cache_k, cache_v, num_splits):
        B = acase.token_position.size
        self.kv, self.B = kv, B
        self.ck, self.cv = dev(cache_k), dev(cache_v)
        self.q = torch.full((B, HQ, D), 0x1234, dtype=torch.int16, device="cuda")
        self.out = torch.full((B, HQ, D), 0x7FC0, dtype=torch.int16, device="cuda")
        self.lse = torch.full((B, HQ), float("nan"), dtype=torch.float32, device="cuda")
        rows = B * HQ * num_splits
        self.pm = torch.full((rows,), float("nan"), dtype=torch.float32, device="cuda")
        self.pl = self.pm.clone()
        self.pacc = torch.full((rows * D,), float("nan"), dtype=torch.float32, device="cuda")
        self.status = torch.zeros(4, dtype=torch.int32, device="cuda")
        self.num_splits = num_splits


def _run_steps(kv, orc, *, window, ring_pages, start, steps, norm_mode, has_v=True, unmapped=None,
               length_of=None, seed=7, page_size=16):
    """start: first position per sequence (-1: never appended). length_of(b, pos) -> seq_length given to
    the attention (default pos + 1)."""
    rng = np.random.default_rng(seed)
    start = np.asarray(start, np.int32)
    B = start.size
    max_pos = int(start.max()) + steps + 1
    acase = helpers.make_append_case(seed, np.maximum(start, 0), window=window, ring_pages=ring_pages,
                                     max_pos=max_pos, has_v=has_v, page_size=page_size)
    if unmapped is not None:
        acase.page_table[unmapped] = -1
    cfg_t = acase.cfg
    cfg = kv.make_kv_config(*cfg_t)
    elems = cfg_t[0] * cfg_t[1] * cfg_t[2] * cfg_t[5] * cfg_t[6]
    ck = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))      # stale rows everywhere
    cv = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    num_splits = kv.plan_balanced(B, sms)
    fused = _State(kv, acase, ck, cv, num_splits)
    plain = _State(kv, acase, ck, cv, num_splits)
    tiled = _State(kv, acase, ck, cv, num_splits)
    ticket = torch.zeros(B * H * kv.TICKETS_PER_HEAD, dtype=torch.int32, device="cuda")
    table, qw, kw_ = dev(acase.page_table), dev(acase.q_w), dev(acase.k_w)
    cos, sin = dev(acase.cos), dev(acase.sin)
    scale = 1.0 / 16.0
    qp_host = np.full((B, HQ, D), 0x1234, np.uint16)
    for t in range(steps):
        pos = np.where(start >= 0, start + t, -1).astype(np.int32)
        length = np.array([(length_of(b, int(p)) if length_of else int(p) + 1) if p >= 0 else 9
                           for b, p in enumerate(pos)], np.int32)
        q = helpers.bf16_normal(rng, (B, HQ, D))
        k = helpers.bf16_normal(rng, (B, H, D))
        v = helpers.bf16_normal(rng, (B, H, D)) if has_v else None
        dq, dk, dv = dev(q), dev(k), (dev(v) if has_v else None)
        dpos, dlen = dev(pos), dev(length)

        a = kv.LayerStepArgs()
        a.q, a.out, a.lse = fused.q.data_ptr(), fused.out.data_ptr(), fused.lse.data_ptr()
        a.partial_m, a.partial_l, a.partial_acc = fused.pm.data_ptr(), fused.pl.data_ptr(), fused.pacc.data_ptr()
        a.cache_k, a.cache_v, a.cache_config = fused.ck.data_ptr(), fused.cv.data_ptr(), cfg
        a.page_table, a.token_position, a.seq_lengths = table.data_ptr(), dpos.data_ptr(), dlen.data_ptr()
        a.cache_layer, a.split_size, a.num_splits, a.softmax_scale = 0, 0, num_splits, scale
        a.raw_q, a.raw_k, a.raw_v = dq.data_ptr(), dk.data_ptr(), (dv.data_ptr() if has_v else None)
        a.q_norm_weight, a.k_norm_weight, a.cos, a.sin = qw.data_ptr(), kw_.data_ptr(), cos.data_ptr(), sin.data_ptr()
        a.batch_count, a.q_heads, a.rotary_dim, a.norm_mode = B, HQ, D, norm_mode
        a.status = fused.status.data_ptr()
        kv.decode_layer_step(a)

        a.q, a.out, a.lse = tiled.q.data_ptr(), tiled.out.data_ptr(), tiled.lse.data_ptr()
        a.partial_m, a.partial_l, a.partial_acc = tiled.pm.data_ptr(), tiled.pl.data_ptr(), tiled.pacc.data_ptr()
        a.cache_k, a.cache_v = tiled.ck.data_ptr(), tiled.cv.data_ptr()
        a.status, a.ticket = tiled.status.data_ptr(), ticket.data_ptr()
        kv.decode_layer_step_tiled(a)

        kv.decode_append(plain.q, plain.ck, plain.cv, cfg, table, dpos, 0, dq, dk, dv, qw, kw_, cos, sin, B, HQ, D,
                         norm_mode)
        kv.decode_attention(plain.out, plain.lse, plain.q, plain.ck, plain.cv, cfg, table, dlen, 0, scale, 0,
                            num_splits, B, HQ, plain.pm, plain.pl, plain.pacc, plain.status)
        torch.cuda.synchronize()
        assert fused.status[0].item() == 0 and plain.status[0].item() == 0

        assert torch.equal(fused.ck, plain.ck) and torch.equal(fused.cv, plain.cv), t
        assert torch.equal(fused.q, plain.q), t
        assert torch.equal(fused.out, plain.out), t
        assert torch.equal(fused.lse.view(torch.int32), plain.lse.view(torch.int32)), t
        assert tiled.status[0].item() == 0 and not ticket.any(), t
        assert torch.equal(tiled.ck, plain.ck) and torch.equal(tiled.cv, plain.cv), t
        assert torch.equal(tiled.q, plain.q), t
        max_abs, max_rel = attention_error(host_u16(tiled.out), orc.bf16_to_f32(host_u16(plain.out)))
        assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (t, max_abs, max_rel)
        la, lb = tiled.lse.cpu().numpy(), plain.lse.cpu().numpy()
        assert np.array_equal(np.isfinite(la), np.isfinite(lb)), t
        assert np.abs(la[np.isfinite(la)] - lb[np.isfinite(lb)]).max(initial=0.0) <= LSE_MAX_ABS, t

        if norm_mode == kv.NORM_IEEE:            # the host oracle states the IEEE arithmetic
            qp = qp_host.copy()
            orc.decode_append(qp, ck, cv, cfg_t, acase.page_table, pos, 0, q, k, v, acase.q_w, acase.k_w,
                              acase.cos, acase.sin, B, HQ, D)
            keep = pos < 0                       # rows of sequences that were not appended stay
            qp[keep] = qp_host[keep]
            qp_host = qp
            if t % 7 == 0 or t == steps - 1:
                assert np.array_equal(host_u16(fused.ck), ck) and np.array_equal(host_u16(fused.cv), cv), t
                assert np.array_equal(host_u16(fused.q), qp.reshape(-1)), t
                ref, ref_lse = orc.decode_attention_f64(qp, ck, cv, acase.page_table, length, cfg_t, 0, scale, B, HQ)
                for which in (fused, tiled):
                    max_abs, max_rel = attention_error(host_u16(which.out), ref)
                    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (t, max_abs, max_rel)
                got_lse = fused.lse.cpu().numpy()
                fin = np.isfinite(ref_lse)
                assert np.array_equal(np.isneginf(got_lse), np.isneginf(ref_lse))
                assert np.abs(got_lse[fin] - ref_lse[fin]).max(initial=0.0) <= LSE_MAX_ABS


@pytest.mark.parametrize("norm", ["ieee", "approx"])
def test_fused_step_sliding_ring_wraps(kv, orc, norm):
    """Window 64 in a tight ring of 4 pages: the ring slot of the new key is the slot of the key that
    just left the window, every step; one sequence is never appended."""
    _run_steps(kv, orc, window=64, ring_pages=4, start=[0, 5, 37, 100, 63, -1], steps=40,
               norm_mode=kv.NORM_IEEE if norm == "ieee" else kv.NORM_RSQRT_APPROX)


def test_fused_step_linear_cache_ragged(kv, orc):
    _run_steps(kv, orc, window=0, ring_pages=None, start=[0, 1, 15, 16, 300, 2047, 777], steps=24,
               norm_mode=kv.NORM_IEEE, seed=11)


def test_fused_step_unmapped_page_and_foreign_lengths(kv, orc):
    """Sequence 1 has no page for positions 32..47: nothing is appended there and the key is not read.
    Sequence 2 is attended with a length that stops before its new position, sequence 3 with length 0:
    their rows are appended all the same, by a CTA that does not stream them."""
    def length_of(b, pos):
        if b == 2:
            return max(pos - 3, 0)
        if b == 3:
            return 0
        return pos + 1
    _run_steps(kv, orc, window=0, ring_pages=None, start=[3, 30, 50, 8], steps=20, norm_mode=kv.NORM_IEEE,
               unmapped=(1, 2), length_of=length_of, seed=13)


def test_fused_step_v_from_raw_k(kv, orc):
    _run_steps(kv, orc, window=64, ring_pages=5, start=[10, 70], steps=12, norm_mode=kv.NORM_IEEE, has_v=False,
               seed=17)


def test_fused_step_batch_one_long_context(kv, orc):
    """Batch 1, 3000 keys: the new key sits in the last of ~190 ranges; everything else streams before it."""
    _run_steps(kv, orc, window=0, ring_pages=None, start=[3000], steps=6, norm_mode=kv.NORM_RSQRT_APPROX, seed=19)


@pytest.mark.parametrize("seed", range(8))
def test_fused_step_random_shapes(kv, orc, seed):
    """Seeded random batches (1..100 sequences, so both with and without idle CTAs), page sizes 4 / 16 / 64,
    sliding and linear caches, a few unmapped pages and skipped sequences: fused and two-launch forms must
    agree bit for bit, and both with the oracle."""
    rng = np.random.default_rng(1000 + seed)
    batch = int(rng.choice([1, 2, 7, 33, 80, 100]))
    page = int(rng.choice([4, 16, 64]))
    window = int(rng.choice([0, 0, 48, 256]))
    hi = 700 if batch <= 33 else 120
    start = rng.integers(0, hi, size=batch).astype(np.int32)
    start[rng.random(batch) < 0.1] = -1
    if (start < 0).all():
        start[0] = 5
    steps = 6
    ring_pages = None if window == 0 else -(-window // page) + int(rng.integers(0, 2))
    acase = helpers.make_append_case(2000 + seed, np.maximum(start, 0), page_size=page, window=window,
                                     ring_pages=ring_pages, max_pos=int(start.max()) + steps + 1)
    unmapped = None
    if rng.random() < 0.5:
        b = int(rng.integers(0, batch))
        unmapped = (b, int(rng.integers(0, acase.page_table.shape[1])))
    _run_steps(kv, orc, window=window, ring_pages=ring_pages, start=start, steps=steps, norm_mode=kv.NORM_IEEE,
               unmapped=unmapped, seed=2000 + seed, page_size=page)
