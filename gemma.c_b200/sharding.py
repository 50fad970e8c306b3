"""Host-side partition of the KV path over the GPUs of one node: numpy front end of the library's C entry points
(b200kv_shard_sequences, b200kv_kv_head_range, b200kv_key_range_page_table; no device code) plus the array slicing
the tests and the bench need around them.

Two ways the path shards, neither of which the single-GPU reference has:
  * by sequence: sequences are independent (own pages, own length, own output rows); each rank owns whole
    sequences and no collective is on the data path;
  * by KV head: heads are independent until the output row is assembled; rank r owns KV heads
    [r * H/N, (r + 1) * H/N) and their query heads, holds a cache with num_heads = H/N, and the step ends with
    an all-gather of the per-head outputs;
  * by key range: rank r owns all heads of the pages of positions [r * C, (r + 1) * C) of one long sequence,
    attends the full query over them, and the ranks' normalised rows are merged with their log-sum-exp
    (b200kv_peer_merge_attention does the exchange and the merge on the GPUs).
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import load_library


def shard_sequences(live_keys, world: int) -> list[list[int]]:
    """Greedy longest-first partition of sequence indices over `world` ranks by live key count
    (b200kv_shard_sequences); a rank's list is in the order the sequences were dealt."""
    keys = np.ascontiguousarray(live_keys, dtype=np.int64)
    owner = np.empty(keys.size, dtype=np.int32)
    if load_library().b200kv_shard_sequences(keys.ctypes.data, keys.size, world, owner.ctypes.data) != 0:
        raise ValueError("b200kv_shard_sequences rejected its arguments")
    order = np.argsort(-keys, kind="stable")
    return [[int(i) for i in order if owner[i] == r] for r in range(world)]


def kv_head_range(kv_heads: int, world: int, rank: int) -> tuple[int, int]:
    first, count = ctypes.c_int32(), ctypes.c_int32()
    if load_library().b200kv_kv_head_range(kv_heads, world, rank, ctypes.byref(first), ctypes.byref(count)) != 0:
        raise ValueError(f"{kv_heads} KV heads do not divide over {world} ranks")
    return first.value, first.value + count.value


def slice_cache_heads(cache: np.ndarray, cfg: tuple, world: int, rank: int):
    """Rank's share of a Layout-A cache [layer, page, offset, head, dim]: the same pages and offsets with
    only its heads. Returns (flat cache, config tuple with num_heads = heads / world)."""
    layers, pages, page_size, mpps, batch, heads, dim, window = cfg
    lo, hi = kv_head_range(heads, world, rank)
    full = np.asarray(cache).reshape(layers, pages, page_size, heads, dim)
    part = np.ascontiguousarray(full[:, :, :, lo:hi, :]).reshape(-1)
    return part, (layers, pages, page_size, mpps, batch, hi - lo, dim, window)


def slice_query_heads(q: np.ndarray, q_heads: int, kv_heads: int, world: int, rank: int) -> np.ndarray:
    """Query rows [batch, q_heads, dim] of the rank's KV heads (GQA groups stay together)."""
    group = q_heads // kv_heads
    lo, hi = kv_head_range(kv_heads, world, rank)
    return np.ascontiguousarray(np.asarray(q)[:, lo * group:hi * group, :])


def key_range_page_table(page_table: np.ndarray, seq_len: int, page_size: int, world: int, rank: int):
    """Rank's view of one sequence's page table for key-range sharding: the pages of its positions moved to the
    front (local positions start at 0), the rest unmapped. Returns (table, local length, first absolute
    position). The keys are dealt in whole pages, the last rank takes the remainder."""
    table = np.ascontiguousarray(page_table, dtype=np.int32)
    assert table.ndim == 2 and table.shape[0] == 1, "one sequence"
    out = np.empty_like(table)
    length, first = ctypes.c_int32(), ctypes.c_int32()
    rc = load_library().b200kv_key_range_page_table(table.ctypes.data, table.shape[1], int(seq_len), page_size, world,
                                                    rank, out.ctypes.data, ctypes.byref(length), ctypes.byref(first))
    if rc != 0:
        raise ValueError("b200kv_key_range_page_table rejected its arguments")
    return out, length.value, first.value


def merge_attention_rows(outs, lses):
    """The merge of b200kv_peer_merge_attention on the host: outs [ranks, rows, dim], lses [ranks, rows]
    (natural log; -inf for a rank without keys). Returns (rows [rows, dim] float64, lse [rows])."""
    outs = np.asarray(outs, dtype=np.float64)
    lses = np.asarray(lses, dtype=np.float64)
    top = lses.max(axis=0)
    safe = np.where(np.isfinite(top), top, 0.0)
    weight = np.exp(lses - safe)
    total = weight.sum(axis=0)
    norm = np.where(total > 0, total, 1.0)
    merged = ((weight / norm)[:, :, None] * np.where(weight[:, :, None] > 0, outs, 0.0)).sum(axis=0)
    with np.errstate(divide="ignore"):
        lse = np.where(total > 0, safe + np.log(norm), -np.inf)
    return merged, lse
