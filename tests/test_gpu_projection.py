"""The decode projections either side of the KV path through the C-ABI:
b200kv_decode_ingress_bf16 (input RMSNorm + [Q|K|V] projection), b200kv_decode_egress_bf16 (O projection +
post-attention norm + residual + pre-FFN norm) and b200kv_decode_attention_layer_bf16 (ingress + layer-step +
egress). The results are bf16 roundings of fp32 sums whose order is the reference block's, so the comparison
is bit for bit: in B200KV_NORM_IEEE mode against the CPU oracle, in the default mode against the
reference's own phases compiled for this GPU (oracle/_ref), when that library is present."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from tests import helpers
from tests.gpu_util import dev, host_u16, need_gpu
from tests.helpers import ATTN_MAX_ABS, ATTN_MAX_REL, attention_error

pytestmark = [pytest.mark.gpu, need_gpu]

HIDDEN = 3840
POISON = 0x7FC0  # bf16 NaN


def _weights(rng, cols, width):
    """Column-major projection matrix with entries ~ N(0, 1/width): outputs of unit scale."""
    return helpers.bf16_normal(rng, (cols, width), std=1.0 / np.sqrt(width))


def _poison(*shape):
    return torch.full(shape, POISON, dtype=torch.int16, device="cuda")


def _ingress_case(seed, rows, cols):
    rng = np.random.default_rng(seed)
    return dict(x=helpers.bf16_normal(rng, (rows, HIDDEN), std=1.7),
                w_in=helpers.bf16_normal(rng, (HIDDEN,), std=0.05, mean=1.0), w=_weights(rng, cols, HIDDEN))


def _run_ingress(kv, case, rows, cols, q_width, k_width, norm_mode):
    raw = _poison(rows * cols)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    keep = [dev(case["x"]), dev(case["w_in"]), dev(case["w"])]
    a = kv.IngressArgs()
    a.raw_qkv, a.x, a.input_norm_weight, a.qkv_proj_col_major = (raw.data_ptr(), keep[0].data_ptr(),
                                                                 keep[1].data_ptr(), keep[2].data_ptr())
    a.batch_count, a.hidden_size, a.cols, a.q_width, a.k_width = rows, HIDDEN, cols, q_width, k_width
    a.norm_mode, a.status = norm_mode, status.data_ptr()
    kv.decode_ingress(a)
    torch.cuda.synchronize()
    assert status[0].item() == 0
    return host_u16(raw), keep


def _segments(raw, rows, cols, q_width, k_width):
    """Row r of the [q | k | v] tensors the ingress lays out one after the other -> [rows, cols]."""
    v_width = cols - q_width - k_width
    q = raw[: rows * q_width].reshape(rows, q_width)
    k = raw[rows * q_width: rows * (q_width + k_width)].reshape(rows, k_width)
    v = raw[rows * (q_width + k_width):].reshape(rows, v_width)
    return np.concatenate([q, k, v], axis=1)


@pytest.mark.parametrize("rows,cols,q_width,k_width", [(1, 8192, 4096, 2048), (3, 8192, 4096, 2048),
                                                        (1, 8704, 8192, 512), (2, 8704, 8192, 512)])
def test_ingress_matches_the_oracle_bit_for_bit(kv, orc, rows, cols, q_width, k_width):
    case = _ingress_case(100 + rows + cols, rows, cols)
    raw, _ = _run_ingress(kv, case, rows, cols, q_width, k_width, kv.NORM_IEEE)
    got = _segments(raw, rows, cols, q_width, k_width)
    for r in range(rows):
        want, _ = orc.decode_ingress(case["x"][r], case["w_in"], case["w"])
        assert np.array_equal(got[r], want), (r, int((got[r] != want).sum()))


def test_ingress_small_and_odd_column_counts(kv, orc):
    """Fewer columns than CTAs x stage, and a count that leaves the last stage of a CTA ragged."""
    for cols in (8, 40, 1096):
        case = _ingress_case(7 + cols, 1, cols)
        raw, _ = _run_ingress(kv, case, 1, cols, cols, 0, kv.NORM_IEEE)
        want, _ = orc.decode_ingress(case["x"][0], case["w_in"], case["w"])
        assert np.array_equal(raw, want), cols


def test_projection_edge_values(kv, orc):
    """A layer input of zeros (the norm's scale is rsqrt(eps), every sum is +0), and inputs of large magnitude
    (sums near the top of bf16's exponent range): still the oracle's bits, ingress and egress."""
    cols, q_width, k_width = 8192, 4096, 2048
    case = _ingress_case(900, 1, cols)
    case["x"] = np.zeros_like(case["x"])
    raw, _ = _run_ingress(kv, case, 1, cols, q_width, k_width, kv.NORM_IEEE)
    assert not raw.any()
    big = _ingress_case(901, 1, cols)
    big["x"] = helpers.bf16_normal(np.random.default_rng(5), (1, HIDDEN), std=3.0e4)
    big["w"] = helpers.bf16_normal(np.random.default_rng(6), (cols, HIDDEN), std=40.0)
    raw, _ = _run_ingress(kv, big, 1, cols, q_width, k_width, kv.NORM_IEEE)
    want, _ = orc.decode_ingress(big["x"][0], big["w_in"], big["w"])
    assert np.array_equal(raw, want) and np.abs(orc.bf16_to_f32(want)).max() > 1.0e3
    ecase = _egress_case(902, 1, 4096)
    ecase["attn"] = np.zeros_like(ecase["attn"])          # O projection of zeros: the residual passes through
    got = _run_egress(kv, ecase, 1, 4096, kv.NORM_IEEE)
    want = orc.decode_egress(ecase["attn"][0], ecase["w_o"], ecase["w_post"], ecase["w_pre"], ecase["x"][0])
    for g, w in zip(got, want):
        assert np.array_equal(g[0], w)
    assert not got[0].any() and np.array_equal(got[2][0], ecase["x"][0])


def _egress_case(seed, rows, width):
    rng = np.random.default_rng(seed)
    return dict(attn=helpers.bf16_normal(rng, (rows, width)), w_o=_weights(rng, HIDDEN, width),
                w_post=helpers.bf16_normal(rng, (HIDDEN,), std=0.05, mean=1.0),
                w_pre=helpers.bf16_normal(rng, (HIDDEN,), std=0.05, mean=1.0),
                x=helpers.bf16_normal(rng, (rows, HIDDEN), std=1.7))


def _run_egress(kv, case, rows, width, norm_mode, with_ffn_x=True, ticket=None, calls=1):
    outs = [_poison(rows, HIDDEN) for _ in range(4)]
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ticket = torch.zeros(rows, dtype=torch.int32, device="cuda") if ticket is None else ticket
    keep = [dev(case[n]) for n in ("attn", "w_o", "w_post", "w_pre", "x")]
    a = kv.EgressArgs()
    a.residual_out, a.normed_out, a.ffn_residual = (t.data_ptr() for t in outs[:3])
    a.ffn_x = outs[3].data_ptr() if with_ffn_x else None
    a.attention_out, a.o_proj_col_major, a.post_norm_weight, a.pre_ffn_norm_weight, a.x = (
        t.data_ptr() for t in keep)
    a.ticket, a.batch_count, a.hidden_size, a.attention_width = ticket.data_ptr(), rows, HIDDEN, width
    a.norm_mode, a.status = norm_mode, status.data_ptr()
    for _ in range(calls):
        kv.decode_egress(a)
    torch.cuda.synchronize()
    assert status[0].item() == 0
    assert int(ticket.abs().sum().item()) == 0, "the ticket must be left at zero"
    return [host_u16(t).reshape(rows, HIDDEN) for t in outs]


@pytest.mark.parametrize("rows,width", [(1, 4096), (2, 4096), (1, 8192), (3, 8192)])
def test_egress_matches_the_oracle_bit_for_bit(kv, orc, rows, width):
    case = _egress_case(200 + rows + width, rows, width)
    got = _run_egress(kv, case, rows, width, kv.NORM_IEEE, calls=3)   # repeated: the ticket is reused
    for r in range(rows):
        want = orc.decode_egress(case["attn"][r], case["w_o"], case["w_post"], case["w_pre"], case["x"][r])
        for name, g, w in zip(("residual_out", "normed_out", "ffn_residual", "ffn_x"), got, want):
            assert np.array_equal(g[r], w), (name, r, int((g[r] != w).sum()))


def test_egress_many_calls_in_a_row_stay_exact(kv, orc):
    """The tail runs in whichever CTA finishes last and reads what all the others wrote: 150 launches back to
    back, outputs poisoned in between, every result the oracle's bits."""
    rows, width = 2, 4096
    case = _egress_case(77, rows, width)
    want = [orc.decode_egress(case["attn"][r], case["w_o"], case["w_post"], case["w_pre"], case["x"][r])
            for r in range(rows)]
    ticket = torch.zeros(rows, dtype=torch.int32, device="cuda")
    for _ in range(15):
        got = _run_egress(kv, case, rows, width, kv.NORM_IEEE, ticket=ticket, calls=10)
        for r in range(rows):
            for g, w in zip(got, want[r]):
                assert np.array_equal(g[r], w)


def test_egress_without_ffn_x_leaves_it_alone(kv, orc):
    case = _egress_case(31, 1, 4096)
    got = _run_egress(kv, case, 1, 4096, kv.NORM_IEEE, with_ffn_x=False)
    want = orc.decode_egress(case["attn"][0], case["w_o"], case["w_post"], case["w_pre"], case["x"][0])
    assert np.array_equal(got[2][0], want[2])
    assert (got[3] == POISON).all()


def test_projection_argument_checks(kv):
    a = kv.IngressArgs()
    assert kv.decode_ingress(a, check=False) == kv.CUDA_SUCCESS          # zero rows: nothing to do
    a.batch_count, a.hidden_size, a.cols, a.q_width = 1, HIDDEN, 8192, 4096
    assert kv.decode_ingress(a, check=False) == kv.CUDA_ERROR_INVALID_VALUE  # null pointers
    e = kv.EgressArgs()
    e.batch_count, e.hidden_size, e.attention_width = 1, HIDDEN, 1000
    assert kv.decode_egress(e, check=False) == kv.CUDA_ERROR_INVALID_VALUE


def _ref():
    from oracle import ref_binding

    if not ref_binding.has_projections():
        pytest.skip("oracle/_ref (the reference's own kernels) is not built here")
    return ref_binding


@pytest.mark.parametrize("global_geometry", [False, True])
def test_default_mode_equals_the_reference_kernels(kv, global_geometry):
    """Default norm mode (rsqrt.approx as in the reference's GPU code) against the reference's own phases on
    the same GPU: raw q/k/v, O projection, both norms and the residual, all bit for bit."""
    ref = _ref()
    cols, q_width, k_width = (8704, 8192, 512) if global_geometry else (8192, 4096, 2048)
    case = _ingress_case(300 + cols, 1, cols)
    raw, keep = _run_ingress(kv, case, 1, cols, q_width, k_width, kv.NORM_RSQRT_APPROX)
    ref_raw, ref_normed = _poison(cols), _poison(HIDDEN)
    assert ref.decode_ingress(ref_raw, ref_normed, keep[0], keep[1], keep[2], global_geometry) == 0
    torch.cuda.synchronize()
    assert np.array_equal(raw, host_u16(ref_raw)), int((raw != host_u16(ref_raw)).sum())

    width = q_width
    ecase = _egress_case(400 + cols, 1, width)
    got = _run_egress(kv, ecase, 1, width, kv.NORM_RSQRT_APPROX)
    outs = [_poison(HIDDEN) for _ in range(4)]
    keep = [dev(ecase[n]) for n in ("attn", "w_o", "w_post", "w_pre", "x")]
    assert ref.decode_egress(*outs, *keep, global_geometry) == 0
    torch.cuda.synchronize()
    for name, g, w in zip(("residual_out", "normed_out", "ffn_residual", "ffn_x"), got, outs):
        assert np.array_equal(g[0], host_u16(w)), (name, int((g[0] != host_u16(w)).sum()))


@pytest.mark.parametrize("rows,window,native_global", [(1, 1024, False), (3, 0, False), (2, 0, True)])
def test_attention_layer_chain(kv, orc, rows, window, native_global):
    """Layer input -> FFN input in one call. Oracle: ingress, append, double-precision attention (tolerance),
    then egress from the attention rows the GPU produced (so the last stage is again compared bit for bit).
    native_global: the reference's global-layer geometry, 16 query heads on one KV head of 512 dims, rotary on
    the first 128, no V projection (V from raw K) -- 8704 projection columns, O projection of width 8192."""
    HQ, H, D, ROT = (16, 1, 512, 128) if native_global else (16, 8, 256, 256)
    q_width, k_width = HQ * D, H * D
    cols = q_width + k_width * (1 if native_global else 2)
    scale = 1.0 / np.sqrt(D)
    rng = np.random.default_rng(500 + rows)
    start = np.array([700, 33, 1500][:rows], np.int32) if window == 0 else np.array([1500][:rows], np.int32)
    acase = helpers.make_append_case(41 + rows, start, window=window, ring_pages=None if window == 0 else 65,
                                     max_pos=int(start.max()) + 2, kv_heads=H, q_heads=HQ, head_dim=D,
                                     rotary_dim=ROT, has_v=not native_global,
                                     theta=1.0e6 if native_global else 1.0e4)
    cfg_t = acase.cfg
    cfg = kv.make_kv_config(*cfg_t)
    elems = cfg_t[0] * cfg_t[1] * cfg_t[2] * cfg_t[5] * cfg_t[6]
    ck = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
    cv = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
    icase = _ingress_case(600 + rows, rows, cols)
    ecase = _egress_case(700 + rows, rows, q_width)
    length = (start + 1).astype(np.int32)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    num_splits = kv.plan_balanced(rows, sms)

    d = {n: dev(v) for n, v in dict(ck=ck, cv=cv, table=acase.page_table, pos=start, length=length, qw=acase.q_w,
                                    kw=acase.k_w, cos=acase.cos, sin=acase.sin, x=icase["x"], w_in=icase["w_in"],
                                    w=icase["w"], w_o=ecase["w_o"], w_post=ecase["w_post"],
                                    w_pre=ecase["w_pre"]).items()}
    q, out = _poison(rows, HQ, D), _poison(rows, HQ, D)
    n_part = rows * HQ * num_splits
    pm = torch.zeros(n_part, dtype=torch.float32, device="cuda")
    pl, pacc = pm.clone(), torch.zeros(n_part * D, dtype=torch.float32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    raw = _poison(rows * cols)
    outs = [_poison(rows, HIDDEN) for _ in range(4)]
    ticket = torch.zeros(rows, dtype=torch.int32, device="cuda")

    a = kv.AttentionLayerArgs()
    s = a.kv
    s.q, s.out, s.lse = q.data_ptr(), out.data_ptr(), None
    s.partial_m, s.partial_l, s.partial_acc = pm.data_ptr(), pl.data_ptr(), pacc.data_ptr()
    s.cache_k, s.cache_v, s.cache_config = d["ck"].data_ptr(), d["cv"].data_ptr(), cfg
    s.page_table, s.token_position, s.seq_lengths = d["table"].data_ptr(), d["pos"].data_ptr(), d["length"].data_ptr()
    s.cache_layer, s.split_size, s.num_splits, s.softmax_scale = 0, 0, num_splits, scale
    s.q_norm_weight, s.k_norm_weight, s.cos, s.sin = (d["qw"].data_ptr(), d["kw"].data_ptr(), d["cos"].data_ptr(),
                                                     d["sin"].data_ptr())
    s.batch_count, s.q_heads, s.rotary_dim, s.norm_mode, s.status = rows, HQ, ROT, kv.NORM_IEEE, status.data_ptr()
    a.attention_x, a.attention_input_norm_weight = d["x"].data_ptr(), d["w_in"].data_ptr()
    a.attention_qkv_proj_col_major, a.attention_o_proj_col_major = d["w"].data_ptr(), d["w_o"].data_ptr()
    a.attention_post_norm_weight, a.attention_pre_ffn_norm_weight = d["w_post"].data_ptr(), d["w_pre"].data_ptr()
    a.raw_qkv = raw.data_ptr()
    a.residual_out, a.normed_out, a.ffn_residual, a.ffn_x = (t.data_ptr() for t in outs)
    a.ticket, a.hidden_size, a.has_v_projection = ticket.data_ptr(), HIDDEN, 0 if native_global else 1
    kv.decode_attention_layer(a)
    torch.cuda.synchronize()
    assert status[0].item() == 0

    raw_rows = np.stack([orc.decode_ingress(icase["x"][r], icase["w_in"], icase["w"])[0] for r in range(rows)])
    rq = np.ascontiguousarray(raw_rows[:, :q_width]).reshape(rows, HQ, D)
    rk = np.ascontiguousarray(raw_rows[:, q_width:q_width + k_width]).reshape(rows, H, D)
    rv = None if native_global else np.ascontiguousarray(raw_rows[:, q_width + k_width:]).reshape(rows, H, D)
    qp = np.zeros((rows, HQ, D), np.uint16)
    orc.decode_append(qp, ck, cv, cfg_t, acase.page_table, start, 0, rq, rk, rv, acase.q_w, acase.k_w, acase.cos,
                      acase.sin, rows, HQ, ROT)
    assert np.array_equal(host_u16(q), qp.reshape(-1))
    assert np.array_equal(host_u16(d["ck"]), ck) and np.array_equal(host_u16(d["cv"]), cv)
    ref, _ = orc.decode_attention_f64(qp, ck, cv, acase.page_table, length, cfg_t, 0, scale, rows, HQ)
    max_abs, max_rel = attention_error(host_u16(out), ref)
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (max_abs, max_rel)
    attn = host_u16(out).reshape(rows, q_width)
    got = [host_u16(t).reshape(rows, HIDDEN) for t in outs]
    for r in range(rows):
        want = orc.decode_egress(attn[r], ecase["w_o"], ecase["w_post"], ecase["w_pre"], icase["x"][r])
        for name, g, w in zip(("residual_out", "normed_out", "ffn_residual", "ffn_x"), got, want):
            assert np.array_equal(g[r], w), (name, r, int((g[r] != w).sum()))


def test_attention_layer_against_the_reference_phases_end_to_end(kv, orc):
    """The whole attention half of a decode layer, this library's one call against the reference's own four
    phases run one after the other on the same GPU (input norm + projection, fused append, split attention +
    reduce at its default split of 20, O projection + norms): raw rows, prepared q and the appended cache rows
    bit for bit (default norm mode = the reference's arithmetic); attention rows within the bf16 band; the
    layer outputs, which inherit the attention rows' last-bit differences through a 4096-term sum, within 2^-6
    of the reference's values (relative to max(|a|, |b|, 1))."""
    ref = _ref()
    HQ, H, D, cols, q_width, k_width = 16, 8, 256, 8192, 4096, 2048
    rng = np.random.default_rng(77)
    start = np.array([1500], np.int32)
    acase = helpers.make_append_case(91, start, window=1024, ring_pages=65, max_pos=1502)
    cfg_t = acase.cfg
    cfg = kv.make_kv_config(*cfg_t)
    elems = cfg_t[0] * cfg_t[1] * cfg_t[2] * cfg_t[5] * cfg_t[6]
    ck = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
    cv = orc.f32_to_bf16(rng.standard_normal(elems, dtype=np.float32))
    icase, ecase = _ingress_case(801, 1, cols), _egress_case(802, 1, q_width)
    length = (start + 1).astype(np.int32)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    num_splits = kv.plan_balanced(1, sms)
    shared = {n: dev(v) for n, v in dict(table=acase.page_table, pos=start, length=length, qw=acase.q_w, kw=acase.k_w,
                                         cos=acase.cos, sin=acase.sin, x=icase["x"], w_in=icase["w_in"], w=icase["w"],
                                         w_o=ecase["w_o"], w_post=ecase["w_post"], w_pre=ecase["w_pre"]).items()}

    def fresh():
        return dict(ck=dev(ck), cv=dev(cv), q=_poison(1, HQ, D), out=_poison(1, HQ, D), raw=_poison(cols),
                    outs=[_poison(HIDDEN) for _ in range(4)])

    mine, theirs = fresh(), fresh()
    pm = torch.zeros(HQ * num_splits, dtype=torch.float32, device="cuda")
    pl, pacc = pm.clone(), torch.zeros(HQ * num_splits * D, dtype=torch.float32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ticket = torch.zeros(1, dtype=torch.int32, device="cuda")
    a = kv.AttentionLayerArgs()
    s = a.kv
    s.q, s.out, s.lse = mine["q"].data_ptr(), mine["out"].data_ptr(), None
    s.partial_m, s.partial_l, s.partial_acc = pm.data_ptr(), pl.data_ptr(), pacc.data_ptr()
    s.cache_k, s.cache_v, s.cache_config = mine["ck"].data_ptr(), mine["cv"].data_ptr(), cfg
    s.page_table, s.token_position, s.seq_lengths = (shared["table"].data_ptr(), shared["pos"].data_ptr(),
                                                     shared["length"].data_ptr())
    s.cache_layer, s.split_size, s.num_splits, s.softmax_scale = 0, 0, num_splits, 1.0 / 16.0
    s.q_norm_weight, s.k_norm_weight, s.cos, s.sin = (shared["qw"].data_ptr(), shared["kw"].data_ptr(),
                                                     shared["cos"].data_ptr(), shared["sin"].data_ptr())
    s.batch_count, s.q_heads, s.rotary_dim, s.norm_mode, s.status = 1, HQ, D, kv.NORM_RSQRT_APPROX, status.data_ptr()
    a.attention_x, a.attention_input_norm_weight = shared["x"].data_ptr(), shared["w_in"].data_ptr()
    a.attention_qkv_proj_col_major, a.attention_o_proj_col_major = shared["w"].data_ptr(), shared["w_o"].data_ptr()
    a.attention_post_norm_weight, a.attention_pre_ffn_norm_weight = shared["w_post"].data_ptr(), shared["w_pre"].data_ptr()
    a.raw_qkv = mine["raw"].data_ptr()
    a.residual_out, a.normed_out, a.ffn_residual, a.ffn_x = (t.data_ptr() for t in mine["outs"])
    a.ticket, a.hidden_size, a.has_v_projection = ticket.data_ptr(), HIDDEN, 1
    kv.decode_attention_layer(a)
    torch.cuda.synchronize()
    assert status[0].item() == 0

    scratch = _poison(HIDDEN)
    assert ref.decode_ingress(theirs["raw"], scratch, shared["x"], shared["w_in"], shared["w"], False) == 0
    raw = theirs["raw"]
    assert ref.decode_append(theirs["q"], theirs["ck"], theirs["cv"], cfg_t, shared["table"], shared["pos"], 0,
                             raw[:q_width], raw[q_width:q_width + k_width], raw[q_width + k_width:], shared["qw"],
                             shared["kw"], shared["cos"], shared["sin"], 1) == 0
    splits = -(-1024 // 20)
    rpm = torch.zeros(HQ * splits, dtype=torch.float32, device="cuda")
    rpl, rpacc = rpm.clone(), torch.zeros(HQ * splits * D, dtype=torch.float32, device="cuda")
    assert ref.decode_attention(theirs["out"], rpm, rpl, rpacc, theirs["q"], theirs["ck"], theirs["cv"],
                                shared["table"], shared["length"], cfg_t, 0, 1.0 / 16.0, 20, splits, 1) == 0
    assert ref.decode_egress(*theirs["outs"], theirs["out"].view(-1), shared["w_o"], shared["w_post"],
                             shared["w_pre"], shared["x"], False) == 0
    torch.cuda.synchronize()

    assert torch.equal(mine["raw"], theirs["raw"])
    assert torch.equal(mine["q"], theirs["q"])
    assert torch.equal(mine["ck"], theirs["ck"]) and torch.equal(mine["cv"], theirs["cv"])
    max_abs, max_rel = attention_error(host_u16(mine["out"]), orc.bf16_to_f32(host_u16(theirs["out"])))
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (max_abs, max_rel)
    for name, m, t in zip(("residual_out", "normed_out", "ffn_residual", "ffn_x"), mine["outs"], theirs["outs"]):
        x, y = orc.bf16_to_f32(host_u16(m)).astype(np.float64), orc.bf16_to_f32(host_u16(t)).astype(np.float64)
        rel = np.abs(x - y) / np.maximum(np.maximum(np.abs(x), np.abs(y)), 1.0)
        assert rel.max() <= 2.0 ** -6, (name, rel.max())
