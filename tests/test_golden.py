"""Golden vectors recorded from the reference's own CUDA kernels on a B200 (tests/golden/*.npz).

CPU part: the host oracle against those vectors -- this is what pins the oracle for the two rows the
reference's test suite leaves unpinned (fused decode append, split/reduce decode attention).
GPU part: the product kernels against the same vectors, and -- where the reference library built from
the gemma.c sources is present -- against the reference kernels run live.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest
import torch

from tests import golden_cases as gc
from tests.helpers import ATTN_MAX_ABS, ATTN_MAX_REL, attention_error

GOLDEN = Path(__file__).resolve().parent / "golden"
have_golden = all((GOLDEN / f"{n}.npz").exists() for n in gc.APPEND_ALL + gc.ATTENTION_ALL)
need_golden = pytest.mark.skipif(not have_golden, reason="golden fixtures not recorded yet")

# The reference's attention accumulates in fp32 with __expf and block-wide tree sums; the oracle restates
# the same order with expf. Both round the result to bf16: they may differ by one bf16 step of the output.
REF_ORDER_MAX_ABS = 2.0 ** -7


def _ulp_close(orc, got_u16, want_u16, max_fraction):
    a = orc.bf16_to_f32(got_u16).astype(np.float64).reshape(-1)
    b = orc.bf16_to_f32(want_u16).astype(np.float64).reshape(-1)
    step = np.maximum(np.abs(b), 2.0 ** -100) * 2.0 ** -7
    assert np.all(np.abs(a - b) <= step), float(np.abs(a - b).max())
    assert (np.asarray(got_u16).reshape(-1) != np.asarray(want_u16).reshape(-1)).mean() <= max_fraction


@need_golden
@pytest.mark.parametrize("name", gc.APPEND_ALL)
def test_oracle_append_against_reference_kernel_output(orc, name):
    """IEEE 1/sqrt on the host vs rsqrt.approx on the GPU: identical except for rare one-step differences."""
    g = np.load(GOLDEN / f"{name}.npz")
    case = gc.build_append(name)
    assert gc.append_digest(case) == str(g["digest"]), "seeded inputs differ from the ones the fixture was recorded with"
    cfg = case.cfg
    elems = cfg[0] * cfg[1] * cfg[2] * cfg[5] * cfg[6]
    ck, cv = np.zeros(elems, np.uint16), np.zeros(elems, np.uint16)
    qp = np.zeros_like(case.q)
    orc.decode_append(qp, ck, cv, cfg, case.page_table, case.token_position, case.layer, case.q, case.k, case.v,
                      case.q_w, case.k_w, case.cos, case.sin, case.token_position.size, case.q_heads, case.rotary_dim)
    row = cfg[5] * cfg[6]
    for b, pos in enumerate(case.token_position):
        phys = int(case.page_table[b, (pos // cfg[2]) % cfg[3]])
        base = orc.cache_offset(cfg, case.layer, phys, int(pos % cfg[2]), 0, 0)
        _ulp_close(orc, ck[base:base + row], g["k_rows"][b], 0.02)
        _ulp_close(orc, cv[base:base + row], g["v_rows"][b], 0.02)
    _ulp_close(orc, qp, g["q_prepared"], 0.02)
    # placement: the reference wrote exactly these rows and nothing else
    assert int((ck != 0).sum()) == int(g["nonzero_k"])


@need_golden
@pytest.mark.parametrize("name", gc.ATTENTION_ALL)
def test_oracle_attention_against_reference_kernel_output(orc, name):
    g = np.load(GOLDEN / f"{name}.npz")
    case, split_size, num_splits = gc.build_attention(name)
    assert gc.attention_digest(case) == str(g["digest"])
    out, *_ = orc.decode_attention_ref(case.q, case.cache_k, case.cache_v, case.page_table, case.seq_lengths,
                                       case.cfg, case.layer, case.scale, split_size, num_splits, case.batch,
                                       case.q_heads)
    max_abs, _ = attention_error(out, orc.bf16_to_f32(g["out"]))
    assert max_abs <= REF_ORDER_MAX_ABS, max_abs
    out64, _ = orc.decode_attention_f64(case.q, case.cache_k, case.cache_v, case.page_table, case.seq_lengths,
                                        case.cfg, case.layer, case.scale, case.batch, case.q_heads)
    max_abs, max_rel = attention_error(g["out"], out64)
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL


gpu = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a CUDA device")]


def _device_append(kv, case, mode):
    from tests.gpu_util import dev, host_u16
    cfg = kv.make_kv_config(*case.cfg)
    ck = torch.zeros(cfg.cache_elements(), dtype=torch.int16, device="cuda")
    cv = torch.zeros_like(ck)
    qp = torch.zeros(case.q.shape, dtype=torch.int16, device="cuda")
    kv.decode_append(qp, ck, cv, cfg, dev(case.page_table), dev(case.token_position), case.layer, dev(case.q),
                     dev(case.k), None if case.v is None else dev(case.v), dev(case.q_w), dev(case.k_w),
                     dev(case.cos), dev(case.sin), case.token_position.size, case.q_heads, case.rotary_dim, mode)
    torch.cuda.synchronize()
    return host_u16(qp), host_u16(ck), host_u16(cv), (qp, ck, cv)


@need_golden
@pytest.mark.parametrize("name", gc.APPEND_ALL)
@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a CUDA device")
def test_product_append_bit_exact_with_reference_kernel_output(kv, orc, name):
    """Default (rsqrt.approx) mode reproduces the reference GPU kernel's cache rows and prepared q bit for bit."""
    g = np.load(GOLDEN / f"{name}.npz")
    case = gc.build_append(name)
    assert gc.append_digest(case) == str(g["digest"])
    qp, ck, cv, _ = _device_append(kv, case, kv.NORM_RSQRT_APPROX)
    cfg = case.cfg
    row = cfg[5] * cfg[6]
    for b, pos in enumerate(case.token_position):
        phys = int(case.page_table[b, (pos // cfg[2]) % cfg[3]])
        base = orc.cache_offset(cfg, case.layer, phys, int(pos % cfg[2]), 0, 0)
        assert np.array_equal(ck[base:base + row], g["k_rows"][b])
        assert np.array_equal(cv[base:base + row], g["v_rows"][b])
    assert np.array_equal(qp, g["q_prepared"].reshape(-1))
    assert int((ck != 0).sum()) == int(g["nonzero_k"])


@need_golden
@pytest.mark.parametrize("name", gc.ATTENTION_ALL)
@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a CUDA device")
def test_product_attention_against_reference_kernel_output(kv, orc, name):
    from tests.gpu_util import dev, host_u16
    g = np.load(GOLDEN / f"{name}.npz")
    case, split_size, num_splits = gc.build_attention(name)
    assert gc.attention_digest(case) == str(g["digest"])
    cfg = kv.make_kv_config(*case.cfg)
    B, H, D = case.batch, case.q_heads, case.head_dim
    if name in gc.ATTENTION_GLOBAL:      # this geometry runs on the balanced partition only
        split_size = 0
        num_splits = kv.plan_balanced(B, torch.cuda.get_device_properties(0).multi_processor_count)
    out = torch.zeros((B, H, D), dtype=torch.int16, device="cuda")
    rows = B * H * num_splits
    pm = torch.zeros(rows, dtype=torch.float32, device="cuda"); pl = torch.zeros_like(pm)
    pacc = torch.zeros(rows * D, dtype=torch.float32, device="cuda")
    kv.decode_attention(out, None, dev(case.q), dev(case.cache_k), dev(case.cache_v), cfg, dev(case.page_table),
                        dev(case.seq_lengths), case.layer, case.scale, split_size, num_splits, B, H, pm, pl, pacc)
    torch.cuda.synchronize()
    max_abs, max_rel = attention_error(host_u16(out), orc.bf16_to_f32(g["out"]))
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (max_abs, max_rel)


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a CUDA device")
def test_product_against_live_reference_kernels(kv, orc):
    """Same inputs through the reference's kernels and through the product, side by side on this GPU:
    cache write and fused append bit-exact, attention within tolerance."""
    from oracle import ref_binding as ref
    from tests import helpers
    from tests.gpu_util import dev, host_u16
    if not ref.available():
        pytest.skip("oracle/_ref/libgemma4_ref.so not built (reference sources not mounted at build time)")
    # fused append, 300 consecutive positions across a ring wrap, batch of 3
    rng = np.random.default_rng(77)
    case = helpers.make_append_case(611, [1000, 5, 1039], window=1024, max_pos=1400)
    cfg = kv.make_kv_config(*case.cfg)
    bufs = {}
    for who in ("ref", "mine"):
        bufs[who] = (torch.zeros(case.q.shape, dtype=torch.int16, device="cuda"),
                     torch.zeros(cfg.cache_elements(), dtype=torch.int16, device="cuda"),
                     torch.zeros(cfg.cache_elements(), dtype=torch.int16, device="cuda"))
    table, qw, kw_, cos, sin = dev(case.page_table), dev(case.q_w), dev(case.k_w), dev(case.cos), dev(case.sin)
    for step in range(300):
        pos = dev((case.token_position + step).astype(np.int32))
        q = dev(helpers.bf16_normal(rng, case.q.shape)); k = dev(helpers.bf16_normal(rng, case.k.shape))
        v = dev(helpers.bf16_normal(rng, case.k.shape))
        assert ref.decode_append(*bufs["ref"], case.cfg, table, pos, 0, q, k, v, qw, kw_, cos, sin, 3) == 0
        kv.decode_append(*bufs["mine"], cfg, table, pos, 0, q, k, v, qw, kw_, cos, sin, 3, 16, 256,
                         kv.NORM_RSQRT_APPROX)
        if step % 50 == 0 or step == 299:
            assert torch.equal(bufs["ref"][0], bufs["mine"][0])
    torch.cuda.synchronize()
    assert torch.equal(bufs["ref"][1], bufs["mine"][1]) and torch.equal(bufs["ref"][2], bufs["mine"][2])
    assert bufs["mine"][1].any()
    # attention over the cache both just built (ring, three sequences), reference split size and ours
    seq = dev((case.token_position + 300).astype(np.int32))
    qd = dev(helpers.bf16_normal(rng, case.q.shape))
    B, H, D = 3, 16, 256
    for split_size, num_splits in ((20, 52), (64, 16)):
        rows = B * H * num_splits
        outs = {}
        for who in ("ref", "mine"):
            out = torch.zeros((B, H, D), dtype=torch.int16, device="cuda")
            pm = torch.zeros(rows, dtype=torch.float32, device="cuda"); pl = torch.zeros_like(pm)
            pacc = torch.zeros(rows * D, dtype=torch.float32, device="cuda")
            if who == "ref":
                assert ref.decode_attention(out, pm, pl, pacc, qd, bufs["ref"][1], bufs["ref"][2], table, seq,
                                            case.cfg, 0, 1 / 16.0, split_size, num_splits, B) == 0
            else:
                kv.decode_attention(out, None, qd, bufs["mine"][1], bufs["mine"][2], cfg, table, seq, 0, 1 / 16.0,
                                    split_size, num_splits, B, H, pm, pl, pacc)
            torch.cuda.synchronize()
            outs[who] = host_u16(out)
        max_abs, max_rel = attention_error(outs["mine"], orc.bf16_to_f32(outs["ref"]))
        assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (max_abs, max_rel)
    # plain cache write
    tb = dev(np.array([0, 1, 2, 2], np.int32)); tp = dev(np.array([3, 1030, 17, 18], np.int32))
    k = dev(helpers.bf16_normal(rng, (4, 8, 256))); v = dev(helpers.bf16_normal(rng, (4, 8, 256)))
    assert ref.kv_cache_write(bufs["ref"][1], bufs["ref"][2], case.cfg, table, tb, tp, 4, 0, k, v) == 0
    kv.kv_cache_write(bufs["mine"][1], bufs["mine"][2], cfg, table, tb, tp, 4, 0, k, v)
    torch.cuda.synchronize()
    assert torch.equal(bufs["ref"][1], bufs["mine"][1]) and torch.equal(bufs["ref"][2], bufs["mine"][2])


have_projection_golden = all((GOLDEN / f"{n}.npz").exists() for n in gc.PROJECTION_ALL)
need_projection_golden = pytest.mark.skipif(not have_projection_golden,
                                            reason="projection fixtures not recorded yet")


@need_projection_golden
@pytest.mark.parametrize("name", gc.PROJECTION_ALL)
def test_oracle_projections_against_reference_kernel_output(orc, name):
    """The host restatement of the block's summation order against what the reference's phases wrote on a
    B200. The O projection has no norm before it: bit for bit. Everything behind a norm may differ by rare
    one-step roundings (IEEE 1/sqrt on the host, rsqrt.approx on the GPU)."""
    g = np.load(GOLDEN / f"{name}.npz")
    case = gc.build_projection(name)
    assert gc.projection_digest(case) == str(g["digest"]), "seeded inputs differ from the recorded ones"
    raw, _ = orc.decode_ingress(case["x"], case["w_in"], case["w_qkv"])
    _ulp_close(orc, raw, g["raw_qkv"], 0.02)
    residual_out, normed_out, ffn_residual, ffn_x = orc.decode_egress(case["attn"], case["w_o"], case["w_post"],
                                                                     case["w_pre"], case["x"])
    assert np.array_equal(residual_out, g["residual_out"])
    _ulp_close(orc, normed_out, g["normed_out"], 0.02)
    _ulp_close(orc, ffn_residual, g["ffn_residual"], 0.02)
    _ulp_close(orc, ffn_x, g["ffn_x"], 0.02)


@need_projection_golden
@pytest.mark.parametrize("name", gc.PROJECTION_ALL)
@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a CUDA device")
def test_product_projections_bit_exact_with_reference_kernel_output(kv, name):
    """Default norm mode: the recorded bits of the reference's kernels, all five rows."""
    from tests.gpu_util import dev, host_u16

    g = np.load(GOLDEN / f"{name}.npz")
    case = gc.build_projection(name)
    d = {n: dev(case[n]) for n in gc.PROJECTION_INPUTS}
    raw = torch.zeros(case["cols"], dtype=torch.int16, device="cuda")
    a = kv.IngressArgs()
    a.raw_qkv, a.x, a.input_norm_weight, a.qkv_proj_col_major = (raw.data_ptr(), d["x"].data_ptr(),
                                                                 d["w_in"].data_ptr(), d["w_qkv"].data_ptr())
    a.batch_count, a.hidden_size, a.cols, a.q_width, a.k_width = 1, gc.HIDDEN, case["cols"], case["q_width"], case["k_width"]
    a.norm_mode = kv.NORM_RSQRT_APPROX
    kv.decode_ingress(a)
    outs = [torch.zeros(gc.HIDDEN, dtype=torch.int16, device="cuda") for _ in range(4)]
    ticket = torch.zeros(1, dtype=torch.int32, device="cuda")
    e = kv.EgressArgs()
    e.residual_out, e.normed_out, e.ffn_residual, e.ffn_x = (t.data_ptr() for t in outs)
    e.attention_out, e.o_proj_col_major, e.post_norm_weight, e.pre_ffn_norm_weight, e.x = (
        d[n].data_ptr() for n in ("attn", "w_o", "w_post", "w_pre", "x"))
    e.ticket, e.batch_count, e.hidden_size, e.attention_width = ticket.data_ptr(), 1, gc.HIDDEN, case["q_width"]
    e.norm_mode = kv.NORM_RSQRT_APPROX
    kv.decode_egress(e)
    torch.cuda.synchronize()
    for n, t in zip(gc.PROJECTION_OUTPUTS, [raw] + outs):
        assert np.array_equal(host_u16(t), g[n]), (n, int((host_u16(t) != g[n]).sum()))
