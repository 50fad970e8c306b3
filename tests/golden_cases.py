"""Seeded cases whose expected outputs were recorded from the reference's own CUDA kernels on a B200
(tests/golden/make_golden.py). Inputs are rebuilt from the seeds; a digest stored with each fixture
guards against the generator drifting."""
from __future__ import annotations

import hashlib

import numpy as np

from tests.helpers import bf16_normal, make_append_case, make_attn_case

GEOM = dict(kv_heads=8, q_heads=16, head_dim=256)    # the geometry the reference's sliding traits are built for

APPEND = {
    "append_cfg1_tight_ring_wrap": dict(seed=9001, positions=[1024], window=1024, ring_pages=64, max_pos=1025),
    "append_slack_ring_wrap": dict(seed=9002, positions=[1040], window=1024, max_pos=1041),
    "append_linear_theta1e6_batch": dict(seed=9003, positions=[0, 15, 16, 4095], window=0, theta=1e6),
    "append_page64": dict(seed=9004, positions=[63, 64, 200], window=0, page_size=64),
}

ATTENTION = {
    # name: (case kwargs, split_size, num_splits)
    "attn_cfg1_tight_ring_wrapped_split20": (dict(seed=9101, seq_lens=[1025], window=1024, ring_pages=64), 20, 52),
    "attn_cfg1_single_split": (dict(seed=9101, seq_lens=[1025], window=1024, ring_pages=64), 1024, 1),
    "attn_linear_4096_split64": (dict(seed=9102, seq_lens=[4096], window=0), 64, 64),
    "attn_mixed_batch_overprovisioned": (dict(seed=9103, seq_lens=[300, 17, 1, 129, 700], window=0), 37, 25),
    "attn_ring_mixed_batch": (dict(seed=9104, seq_lens=[5000, 90, 1024, 1025], window=1024), 20, 52),
    "attn_page64_straddle": (dict(seed=9105, seq_lens=[1000, 65], window=0, page_size=64), 20, 50),
    "attn_outliers": (dict(seed=9106, seq_lens=[3000], window=0, outlier_frac=0.01), 128, 24),
}


# The reference's native global-layer geometry (src/gemma4.h:19-21,28): 16 query heads on one KV head of
# 512 dims, rotary on the first 128 dims, V = scale-free norm of raw K (no V projection).
GEOM_GLOBAL = dict(kv_heads=1, q_heads=16, head_dim=512)

APPEND_GLOBAL = {
    "append_global_linear_batch": dict(seed=9201, positions=[0, 15, 16, 4095], window=0, theta=1e6),
    "append_global_page64": dict(seed=9202, positions=[63, 64, 200], window=0, page_size=64, theta=1e6),
}

ATTENTION_GLOBAL = {
    "attn_global_4096_page64_split64": (dict(seed=9301, seq_lens=[4096], window=0, page_size=64), 64, 64),
    "attn_global_mixed_batch": (dict(seed=9302, seq_lens=[300, 17, 1, 129, 700], window=0), 37, 25),
    "attn_global_outliers": (dict(seed=9303, seq_lens=[3000], window=0, outlier_frac=0.01), 128, 24),
}

APPEND_ALL = list(APPEND) + list(APPEND_GLOBAL)
ATTENTION_ALL = list(ATTENTION) + list(ATTENTION_GLOBAL)


def build_append(name):
    if name in APPEND_GLOBAL:
        kw = dict(APPEND_GLOBAL[name])
        seed = kw.pop("seed")
        return make_append_case(seed, **kw, **GEOM_GLOBAL, rotary_dim=128, has_v=False)
    kw = dict(APPEND[name])
    seed = kw.pop("seed")
    return make_append_case(seed, **kw, **GEOM)


def build_attention(name):
    table, geom = (ATTENTION_GLOBAL, GEOM_GLOBAL) if name in ATTENTION_GLOBAL else (ATTENTION, GEOM)
    kw, split_size, num_splits = table[name]
    kw = dict(kw)
    seed = kw.pop("seed")
    return make_attn_case(seed, **kw, **geom), split_size, num_splits


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        if a is not None:
            h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def append_digest(case) -> str:
    return digest(case.page_table, case.token_position, case.q, case.k, case.v, case.q_w, case.k_w, case.cos, case.sin)


def attention_digest(case) -> str:
    return digest(case.page_table, case.seq_lengths, case.q, case.cache_k, case.cache_v)


# The decode projections either side of the KV path (src/gemma4_flash_attention_decode.cu:35-129,447-496),
# one row, hidden size 3840, for the reference's two geometries.
HIDDEN = 3840
PROJECTION = {
    "proj_sliding": dict(seed=9401, cols=8192, q_width=4096, k_width=2048, global_geometry=False),
    "proj_global": dict(seed=9402, cols=8704, q_width=8192, k_width=512, global_geometry=True),
}
PROJECTION_ALL = list(PROJECTION)
PROJECTION_INPUTS = ("x", "w_in", "w_qkv", "attn", "w_o", "w_post", "w_pre")
PROJECTION_OUTPUTS = ("raw_qkv", "residual_out", "normed_out", "ffn_residual", "ffn_x")


def build_projection(name) -> dict:
    kw = PROJECTION[name]
    rng = np.random.default_rng(kw["seed"])
    width = kw["q_width"]
    return dict(
        x=bf16_normal(rng, (HIDDEN,), std=1.7),
        w_in=bf16_normal(rng, (HIDDEN,), std=0.05, mean=1.0),
        w_qkv=bf16_normal(rng, (kw["cols"], HIDDEN), std=1.0 / np.sqrt(HIDDEN)),
        attn=bf16_normal(rng, (width,)),
        w_o=bf16_normal(rng, (HIDDEN, width), std=1.0 / np.sqrt(width)),
        w_post=bf16_normal(rng, (HIDDEN,), std=0.05, mean=1.0),
        w_pre=bf16_normal(rng, (HIDDEN,), std=0.05, mean=1.0),
        **{k: kw[k] for k in ("cols", "q_width", "k_width", "global_geometry")})


def projection_digest(case) -> str:
    return digest(*(case[n] for n in PROJECTION_INPUTS))
