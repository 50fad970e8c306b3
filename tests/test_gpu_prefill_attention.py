"""Prompt attention -- the two entry points of src/gemma4_flash_attention.cuh -- through the C-ABI:
causal (+ sliding window) attention of each sequence over its own prepared rows against the
double-precision oracle (stated bf16 tolerance), and the full calls (prep + attention) with the
prepared rows bit-identical to the stand-alone prep."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from tests import helpers
from tests.gpu_util import dev, host_u16, need_gpu
from tests.helpers import ATTN_MAX_ABS, ATTN_MAX_REL, attention_error

pytestmark = [pytest.mark.gpu, need_gpu]

SLIDING = dict(q_heads=16, kv_heads=8, head_dim=256)
GLOBAL = dict(q_heads=16, kv_heads=1, head_dim=512)


def _rows(rng, batch, seq, q_heads, kv_heads, head_dim, k_outliers=False):
    q = helpers.bf16_normal(rng, (batch * seq, q_heads, head_dim))
    k = helpers.bf16_normal(rng, (batch * seq, kv_heads, head_dim))
    v = helpers.bf16_normal(rng, (batch * seq, kv_heads, head_dim))
    return q, k, v


@pytest.mark.parametrize("name,geom,batch,seq,window", [
    ("sliding_window_inside", SLIDING, 2, 200, 64),
    ("sliding_window_larger_than_prompt", SLIDING, 1, 333, 1024),
    ("sliding_one_block_exact", SLIDING, 3, 64, 16),
    ("sliding_single_token", SLIDING, 2, 1, 1024),
    ("sliding_block_plus_one", SLIDING, 1, 65, 7),
    ("sliding_window_one", SLIDING, 1, 100, 1),
    ("global_causal", GLOBAL, 2, 150, 0),
    ("global_block_edges", GLOBAL, 1, 129, 0),
])
def test_prefill_attention_against_double_precision(kv, orc, name, geom, batch, seq, window):
    rng = np.random.default_rng(hash(name) % (2 ** 31))
    q, k, v = _rows(rng, batch, seq, **geom)
    H, HKV, D = geom["q_heads"], geom["kv_heads"], geom["head_dim"]
    scale = 1.0 / np.sqrt(D)
    out = torch.full((batch * seq, H, D), 0x7FC0, dtype=torch.int16, device="cuda")
    kv.prefill_attention(out, dev(q), dev(k), dev(v), batch, seq, H, HKV, D, window, scale)
    torch.cuda.synchronize()
    assert kv.prefill_attention_fault() == 0
    ref, _ = orc.prefill_attention_f64(q, k, v, batch, seq, H, HKV, D, window, scale)
    got = host_u16(out)
    assert not np.isnan(orc.bf16_to_f32(got)).any()
    max_abs, max_rel = attention_error(got, ref)
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (max_abs, max_rel)


def test_sliding_entry_point_preps_then_attends(kv, orc):
    """gemma4_flash_attention_sliding_fwd_bf16_norm_rope: prepared rows are those of the stand-alone prep
    (same kernel, reference GPU arithmetic), attention as the oracle on those rows."""
    rng = np.random.default_rng(31)
    batch, seq, window = 2, 180, 96
    H, HKV, D = 16, 8, 256
    q, k, v = _rows(rng, batch, seq, H, HKV, D)
    qw = helpers.bf16_normal(rng, (D,), std=0.05, mean=1.0)
    kw_ = helpers.bf16_normal(rng, (D,), std=0.05, mean=1.0)
    cos, sin = orc.fill_rope_tables(seq, D // 2, 10000.0, D)
    pos = np.tile(np.arange(seq, dtype=np.int32), batch)
    scale = 1.0 / 16.0
    bufs = [torch.zeros((batch * seq, h, D), dtype=torch.int16, device="cuda") for h in (H, H, HKV, HKV)]
    out, qp, kp, vp = bufs
    args = (dev(q), dev(k), dev(v), dev(qw), dev(kw_), dev(cos), dev(sin), dev(pos))
    kv.flash_attention_sliding_fwd(out, qp, kp, vp, *args, batch, seq, seq, window, scale)
    qp2, kp2, vp2 = (torch.zeros_like(t) for t in (qp, kp, vp))
    kv.prefill_prep(qp2, kp2, vp2, *args, batch * seq, H, HKV, D, D, kv.NORM_RSQRT_APPROX)
    torch.cuda.synchronize()
    assert torch.equal(qp, qp2) and torch.equal(kp, kp2) and torch.equal(vp, vp2)
    ref, _ = orc.prefill_attention_f64(host_u16(qp).reshape(-1, H, D), host_u16(kp).reshape(-1, HKV, D),
                                       host_u16(vp).reshape(-1, HKV, D), batch, seq, H, HKV, D, window, scale)
    max_abs, max_rel = attention_error(host_u16(out), ref)
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (max_abs, max_rel)
    # argument contract of src/gemma4_flash_attention_prefill.cu:1131-1139
    assert kv.flash_attention_sliding_fwd(out, qp, kp, vp, *args, batch, seq, seq + 1, window, scale,
                                          check=False) == kv.CUDA_ERROR_INVALID_VALUE
    assert kv.flash_attention_sliding_fwd(out, qp, kp, vp, *args, batch, seq, seq, 0, scale,
                                          check=False) == kv.CUDA_ERROR_INVALID_VALUE
    assert kv.flash_attention_sliding_fwd(out, qp, kp, vp, *args[:-1], None, batch, seq, seq, window, scale,
                                          check=False) == kv.CUDA_ERROR_INVALID_VALUE


def test_global_entry_point_preps_then_attends(kv, orc):
    """gemma4_flash_attention_global_fwd_bf16_norm_rope: 1 KV head x 512, rotary 128, V from raw K."""
    rng = np.random.default_rng(32)
    batch, seq = 2, 140
    H, HKV, D, ROT = 16, 1, 512, 128
    q = helpers.bf16_normal(rng, (batch * seq, H, D))
    k = helpers.bf16_normal(rng, (batch * seq, HKV, D))
    qw = helpers.bf16_normal(rng, (D,), std=0.05, mean=1.0)
    kw_ = helpers.bf16_normal(rng, (D,), std=0.05, mean=1.0)
    cos, sin = orc.fill_rope_tables(seq, ROT // 2, 1.0e6, D)
    pos = np.tile(np.arange(seq, dtype=np.int32), batch)
    scale = 1.0 / np.sqrt(D)
    out, qp = (torch.zeros((batch * seq, H, D), dtype=torch.int16, device="cuda") for _ in range(2))
    kp, vp = (torch.zeros((batch * seq, HKV, D), dtype=torch.int16, device="cuda") for _ in range(2))
    dq, dk, dqw, dkw, dcos, dsin, dpos = dev(q), dev(k), dev(qw), dev(kw_), dev(cos), dev(sin), dev(pos)
    kv.flash_attention_global_fwd(out, qp, kp, vp, dq, dk, dqw, dkw, dcos, dsin, dpos, batch, seq, seq, scale)
    qp2, kp2, vp2 = (torch.zeros_like(t) for t in (qp, kp, vp))
    kv.prefill_prep(qp2, kp2, vp2, dq, dk, None, dqw, dkw, dcos, dsin, dpos, batch * seq, H, HKV, D, ROT,
                    kv.NORM_RSQRT_APPROX)
    torch.cuda.synchronize()
    assert torch.equal(qp, qp2) and torch.equal(kp, kp2) and torch.equal(vp, vp2)
    ref, _ = orc.prefill_attention_f64(host_u16(qp).reshape(-1, H, D), host_u16(kp).reshape(-1, HKV, D),
                                       host_u16(vp).reshape(-1, HKV, D), batch, seq, H, HKV, D, 0, scale)
    max_abs, max_rel = attention_error(host_u16(out), ref)
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (max_abs, max_rel)


@pytest.mark.parametrize("kind,batch,seq,window", [("sliding", 2, 300, 128), ("sliding", 1, 1100, 1024),
                                                   ("global", 2, 200, 0)])
def test_entry_points_against_live_reference_kernels(kv, orc, kind, batch, seq, window):
    """The same call through the reference's own entry point (its sources compiled for this GPU) and through
    the library: prepared q/k/v identical bit for bit, attention rows within the bf16 tolerance."""
    from oracle import ref_binding as ref
    if not ref.has_prefill():
        pytest.skip("oracle/_ref was built without the reference's prompt attention")
    rng = np.random.default_rng(97)
    H = 16
    HKV, D, ROT, theta = (8, 256, 256, 1.0e4) if kind == "sliding" else (1, 512, 128, 1.0e6)
    q = helpers.bf16_normal(rng, (batch * seq, H, D))
    k = helpers.bf16_normal(rng, (batch * seq, HKV, D))
    v = helpers.bf16_normal(rng, (batch * seq, HKV, D))
    qw = helpers.bf16_normal(rng, (D,), std=0.05, mean=1.0)
    kw_ = helpers.bf16_normal(rng, (D,), std=0.05, mean=1.0)
    cos, sin = orc.fill_rope_tables(seq, ROT // 2, theta, D)
    pos = np.tile(np.arange(seq, dtype=np.int32), batch)
    scale = 1.0 / np.sqrt(D)
    dq, dk, dv, dqw, dkw, dcos, dsin, dpos = (dev(x) for x in (q, k, v, qw, kw_, cos, sin, pos))
    res = {}
    for who in ("ref", "mine"):
        out, qp = (torch.zeros((batch * seq, H, D), dtype=torch.int16, device="cuda") for _ in range(2))
        kp, vp = (torch.zeros((batch * seq, HKV, D), dtype=torch.int16, device="cuda") for _ in range(2))
        if kind == "sliding":
            if who == "ref":
                assert ref.prefill_sliding(out, qp, kp, vp, dq, dk, dv, dqw, dkw, dcos, dsin, dpos, batch, seq, seq,
                                           window, scale) == 0
            else:
                kv.flash_attention_sliding_fwd(out, qp, kp, vp, dq, dk, dv, dqw, dkw, dcos, dsin, dpos, batch, seq,
                                               seq, window, scale)
        else:
            if who == "ref":
                assert ref.prefill_global(out, qp, kp, vp, dq, dk, dqw, dkw, dcos, dsin, dpos, batch, seq, seq,
                                          scale) == 0
            else:
                kv.flash_attention_global_fwd(out, qp, kp, vp, dq, dk, dqw, dkw, dcos, dsin, dpos, batch, seq, seq,
                                              scale)
        torch.cuda.synchronize()
        res[who] = (out, qp, kp, vp)
    for i in (1, 2, 3):
        assert torch.equal(res["ref"][i], res["mine"][i]), ("prepared", i)
    max_abs, max_rel = attention_error(host_u16(res["mine"][0]), orc.bf16_to_f32(host_u16(res["ref"][0])))
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (max_abs, max_rel)


@pytest.mark.parametrize("geom,batch,seq,window", [(SLIDING, 2, 2048, 1024), (SLIDING, 3, 700, 0),
                                                   (GLOBAL, 1, 2048, 0), (GLOBAL, 2, 900, 256)])
def test_prefill_attention_repeats_without_a_wait_running_out(kv, geom, batch, seq, window):
    """Many key tiles per CTA and many calls: every bounded wait of the tensor-core kernel is met (the fault
    word stays 0 -- a role running a barrier phase ahead of its reader would show here) and the result is
    the same bits every time."""
    rng = np.random.default_rng(seq)
    q, k, v = _rows(rng, batch, seq, **geom)
    H, HKV, D = geom["q_heads"], geom["kv_heads"], geom["head_dim"]
    dq, dk, dv = dev(q), dev(k), dev(v)
    first = None
    for _ in range(40):
        out = torch.full((batch * seq, H, D), 0x7FC0, dtype=torch.int16, device="cuda")
        kv.prefill_attention(out, dq, dk, dv, batch, seq, H, HKV, D, window, D ** -0.5)
        torch.cuda.synchronize()
        assert kv.prefill_attention_fault() == 0
        if first is None:
            first = out
        else:
            assert torch.equal(out, first)


def test_prefill_attention_last_tiles_are_waited_for(kv):
    """1500 calls on prompts whose last query block is the longest CTA and the first one launched (cold loads):
    the final wait of the softmax warps must cover the last two P V products, not just the parity of the last
    (it passed early about once in 2000 calls before it waited one phase at a time; the symptom was one block of
    rows divided by an incomplete row sum). Every call must give the first call's bits."""
    rng = np.random.default_rng(5)
    batch, seq, window = 3, 700, 0
    q, k, v = _rows(rng, batch, seq, **SLIDING)
    H, HKV, D = SLIDING["q_heads"], SLIDING["kv_heads"], SLIDING["head_dim"]
    dq, dk, dv = dev(q), dev(k), dev(v)
    first = None
    for _ in range(1500):
        out = torch.full((batch * seq, H, D), 0x7FC0, dtype=torch.int16, device="cuda")
        kv.prefill_attention(out, dq, dk, dv, batch, seq, H, HKV, D, window, D ** -0.5)
        if first is None:
            first = out
        else:
            assert torch.equal(out, first)
    assert kv.prefill_attention_fault() == 0


@pytest.mark.parametrize("geom,batch,seq,window", [(SLIDING, 2, 1500, 1024), (GLOBAL, 1, 1300, 0)])
def test_prefill_attention_long_prompt_against_torch_fp32(kv, orc, geom, batch, seq, window):
    """Prompts too long for the double-precision host oracle in a test: plain fp32 torch attention on the same
    bf16 rows as the reference, same tolerance."""
    rng = np.random.default_rng(seq + 1)
    q, k, v = _rows(rng, batch, seq, **geom)
    H, HKV, D = geom["q_heads"], geom["kv_heads"], geom["head_dim"]
    scale = D ** -0.5
    dq, dk, dv = dev(q), dev(k), dev(v)
    out = torch.full((batch * seq, H, D), 0x7FC0, dtype=torch.int16, device="cuda")
    kv.prefill_attention(out, dq, dk, dv, batch, seq, H, HKV, D, window, scale)
    torch.cuda.synchronize()
    assert kv.prefill_attention_fault() == 0

    def f32(t, heads):
        return t.view(torch.bfloat16).float().view(batch, seq, heads, D).transpose(1, 2)
    qf, kf, vf = f32(dq, H), f32(dk, HKV).repeat_interleave(H // HKV, 1), f32(dv, HKV).repeat_interleave(H // HKV, 1)
    s = qf @ kf.transpose(-1, -2) * scale
    r = torch.arange(seq, device="cuda")[:, None]
    c = torch.arange(seq, device="cuda")[None, :]
    mask = c > r
    if window > 0:
        mask |= c < r - window + 1
    s.masked_fill_(mask, float("-inf"))
    ref = (torch.softmax(s, -1) @ vf).transpose(1, 2).reshape(batch * seq, H, D).cpu().numpy().astype(np.float64)
    max_abs, max_rel = attention_error(host_u16(out), ref)
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (max_abs, max_rel)
