"""Seeded synthetic cases shared by the CPU and GPU tests.

Everything is numpy; bf16 tensors are uint16 bit patterns. The GPU tests move
these arrays to the device unchanged and hand raw pointers to the C-ABI.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np

from oracle import binding as orc


def bf16_normal(rng: np.random.Generator, shape, std: float = 1.0, mean: float = 0.0) -> np.ndarray:
    return orc.f32_to_bf16((rng.standard_normal(shape, dtype=np.float32) * std + mean).astype(np.float32))


def closed_form_value(seed: np.ndarray, mul: int = 37, add: int = 17, div: float = 64.0) -> np.ndarray:
    """The reference tests' fixture-free generator, e.g. tests/test_kv_cache.cu:42-45:
    (((seed * 37 + 17) % 257) - 128) / 64 rounded to bf16."""
    seed = np.asarray(seed, dtype=np.int64)
    centered = ((seed * mul + add) % 257) - 128
    return orc.f32_to_bf16((centered.astype(np.float32) / np.float32(div)))


@dataclass
class AttnCase:
    cfg: tuple            # the eight Gemma4KvCacheConfig fields
    layer: int
    q_heads: int
    page_table: np.ndarray    # int32 [batch, max_pages_per_seq]
    seq_lengths: np.ndarray   # int32 [batch]
    q: np.ndarray             # uint16 [batch, q_heads, D] (prepared)
    cache_k: np.ndarray       # uint16 flat Layout-A
    cache_v: np.ndarray
    scale: float
    extra: dict = field(default_factory=dict)

    @property
    def batch(self) -> int:
        return int(self.seq_lengths.size)

    @property
    def head_dim(self) -> int:
        return self.cfg[6]

    @property
    def kv_heads(self) -> int:
        return self.cfg[5]


def build_page_table(rng, batch, max_pages_per_seq, pages_needed, permute=True, num_pages=None):
    """Page table over one shared pool. pages_needed[b] slots are mapped per sequence
    (slots 0..n-1), the rest stay -1. Physical pages are a seeded permutation of the pool."""
    total = int(sum(pages_needed))
    if num_pages is None:
        num_pages = total
    assert num_pages >= total
    pool = rng.permutation(num_pages).astype(np.int32) if permute else np.arange(num_pages, dtype=np.int32)
    table = np.full((batch, max_pages_per_seq), -1, dtype=np.int32)
    cursor = 0
    for b in range(batch):
        n = int(pages_needed[b])
        table[b, :n] = pool[cursor:cursor + n]
        cursor += n
    return table, num_pages


def make_attn_case(seed, seq_lens, page_size=16, kv_heads=8, q_heads=16, head_dim=256, window=0,
                   ring_pages=None, layers=1, layer=0, permute=True, outlier_frac=0.0, outlier_scale=8.0,
                   extra_pages=0, q_std=1.0) -> AttnCase:
    """Random prepared-looking q and cache contents for a batch of sequences.

    window == 0: linear cache sized for the longest sequence. window > 0: ring of `ring_pages` slots
    (default: the runtime's window + one page of slack, src/gemma4_runtime.cu:18-24)."""
    rng = np.random.default_rng(seed)
    seq_lens = np.asarray(seq_lens, dtype=np.int32)
    batch = seq_lens.size
    if window > 0:
        mpps = ring_pages if ring_pages is not None else -(-(window + page_size - 1) // page_size)
        needed = [min(mpps, -(-max(int(s), 1) // page_size)) for s in seq_lens]
    else:
        mpps = max(1, -(-int(seq_lens.max(initial=1)) // page_size))
        needed = [-(-max(int(s), 0) // page_size) for s in seq_lens]
    table, num_pages = build_page_table(rng, batch, mpps, needed, permute=permute,
                                        num_pages=int(sum(needed)) + extra_pages)
    num_pages = max(num_pages, 1)
    cfg = (layers, num_pages, page_size, mpps, batch, kv_heads, head_dim, window)
    elems = layers * num_pages * page_size * kv_heads * head_dim
    k = rng.standard_normal(elems, dtype=np.float32)
    v = rng.standard_normal(elems, dtype=np.float32)
    if outlier_frac > 0:
        rows = k.reshape(-1, head_dim)
        pick = rng.random(rows.shape[0]) < outlier_frac
        rows[pick] *= outlier_scale
    q = bf16_normal(rng, (batch, q_heads, head_dim), std=q_std)
    return AttnCase(cfg=cfg, layer=layer, q_heads=q_heads, page_table=table, seq_lengths=seq_lens.copy(),
                    q=q, cache_k=orc.f32_to_bf16(k), cache_v=orc.f32_to_bf16(v),
                    scale=1.0 / math.sqrt(head_dim))


def attention_error(out_bf16: np.ndarray, ref_f32: np.ndarray):
    """max_abs and max_rel with the reference bench's denominator max(|a|,|b|,1)
    (src/benches/gemma4_bench_utils.cuh:450-472)."""
    a = orc.bf16_to_f32(out_bf16).astype(np.float64).reshape(-1)
    b = ref_f32.astype(np.float64).reshape(-1)
    diff = np.abs(a - b)
    denom = np.maximum(np.maximum(np.abs(a), np.abs(b)), 1.0)
    return float(diff.max(initial=0.0)), float((diff / denom).max(initial=0.0))


# Stated tolerances for decode attention against the double-precision oracle on the same bf16 cache.
ATTN_MAX_ABS = 2.0 ** -6
ATTN_MAX_REL = 2.0 ** -6
LSE_MAX_ABS = 1.0e-3


@dataclass
class AppendCase:
    cfg: tuple
    layer: int
    q_heads: int
    rotary_dim: int
    page_table: np.ndarray
    token_position: np.ndarray   # int32 [batch]
    q: np.ndarray                # raw [batch, q_heads, D]
    k: np.ndarray                # raw [batch, kv_heads, D]
    v: np.ndarray | None
    q_w: np.ndarray
    k_w: np.ndarray
    cos: np.ndarray
    sin: np.ndarray


def make_append_case(seed, positions, page_size=16, kv_heads=8, q_heads=16, head_dim=256, rotary_dim=256,
                     window=1024, ring_pages=None, layers=1, layer=0, theta=10000.0, exponent_dim=None,
                     has_v=True, weight_std=0.05, permute=True, max_pos=None) -> AppendCase:
    rng = np.random.default_rng(seed)
    positions = np.asarray(positions, dtype=np.int32)
    batch = positions.size
    top = int(max(positions.max(initial=0), 0)) + 1
    if max_pos is None:
        max_pos = top
    if window > 0:
        mpps = ring_pages if ring_pages is not None else -(-(window + page_size - 1) // page_size)
    else:
        mpps = max(1, -(-max_pos // page_size))
    needed = [min(mpps, -(-max_pos // page_size))] * batch
    table, num_pages = build_page_table(rng, batch, mpps, needed, permute=permute)
    cfg = (layers, max(num_pages, 1), page_size, mpps, batch, kv_heads, head_dim, window)
    cos, sin = orc.fill_rope_tables(max_pos, rotary_dim // 2, theta, exponent_dim or head_dim)
    return AppendCase(
        cfg=cfg, layer=layer, q_heads=q_heads, rotary_dim=rotary_dim, page_table=table,
        token_position=positions.copy(),
        q=bf16_normal(rng, (batch, q_heads, head_dim)), k=bf16_normal(rng, (batch, kv_heads, head_dim)),
        v=bf16_normal(rng, (batch, kv_heads, head_dim)) if has_v else None,
        q_w=bf16_normal(rng, (head_dim,), std=weight_std, mean=1.0),
        k_w=bf16_normal(rng, (head_dim,), std=weight_std, mean=1.0),
        cos=cos, sin=sin)
