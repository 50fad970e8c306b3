"""CPU checks of the oracle's decode projections (oracle/kv_oracle.cpp: orc_decode_ingress / orc_decode_egress):
the block-order sums against plain double-precision arithmetic, and the pieces against each other."""
from __future__ import annotations

import numpy as np

from tests import golden_cases as gc


def _f64(orc, a):
    return orc.bf16_to_f32(a).astype(np.float64)


def _rms(orc, x, w):
    v = _f64(orc, x)
    return v / np.sqrt((v * v).mean() + 1e-6) * _f64(orc, w)


def _one_step(orc, got, want_f64):
    """Within one bf16 rounding step of a double-precision value."""
    g = _f64(orc, got)
    assert np.all(np.abs(g - want_f64) <= np.maximum(np.abs(want_f64), 2.0 ** -20) * 2.0 ** -7)


def test_ingress_is_norm_then_projection(orc):
    case = gc.build_projection("proj_sliding")
    raw, normed = orc.decode_ingress(case["x"], case["w_in"], case["w_qkv"], threads=4)
    assert np.array_equal(normed, orc.hidden_rmsnorm(case["x"], case["w_in"]))
    _one_step(orc, normed, _rms(orc, case["x"], case["w_in"]))
    want = _f64(orc, case["w_qkv"]) @ _f64(orc, normed)
    got = _f64(orc, raw)
    # fp32 accumulation of 3840 products of unit-scale values, then one bf16 rounding
    assert np.abs(got - want).max() <= 2.0 ** -7 * max(1.0, np.abs(want).max())
    assert raw.shape == (8192,)


def test_egress_chain(orc):
    case = gc.build_projection("proj_global")
    o, normed, ffn_residual, ffn_x = orc.decode_egress(case["attn"], case["w_o"], case["w_post"], case["w_pre"],
                                                       case["x"], threads=4)
    want = _f64(orc, case["w_o"]) @ _f64(orc, case["attn"])
    assert np.abs(_f64(orc, o) - want).max() <= 2.0 ** -7 * max(1.0, np.abs(want).max())
    _one_step(orc, normed, _rms(orc, o, case["w_post"]))
    _one_step(orc, ffn_residual, _f64(orc, case["x"]) + _f64(orc, normed))
    _one_step(orc, ffn_x, _rms(orc, ffn_residual, case["w_pre"]))


def test_projection_is_independent_of_host_threads(orc):
    case = gc.build_projection("proj_sliding")
    a, _ = orc.decode_ingress(case["x"], case["w_in"], case["w_qkv"], threads=1)
    b, _ = orc.decode_ingress(case["x"], case["w_in"], case["w_qkv"], threads=7)
    assert np.array_equal(a, b)
