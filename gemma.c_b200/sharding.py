"""Host-side partition of the KV path over the GPUs of one node (numpy only, no device code).

Two ways the path shards, neither of which the single-GPU reference has:
  * by sequence: sequences are independent (own pages, own length, own output rows); each rank owns whole
    sequences and no collective is on the data path;
  * by KV head: heads are independent until the output row is assembled; rank r owns KV heads
    [r * H/N, (r + 1) * H/N) and their query heads, holds a cache with num_heads = H/N, and the step ends with
    an all-gather of the per-head outputs.
"""
from __future__ import annotations

import numpy as np


def shard_sequences(live_keys, world: int) -> list[list[int]]:
    """Greedy longest-first partition of sequence indices over `world` ranks by live key count."""
    keys = np.asarray(live_keys, dtype=np.int64)
    order = np.argsort(-keys, kind="stable")
    load = [0] * world
    shards: list[list[int]] = [[] for _ in range(world)]
    for i in order:
        r = int(np.argmin(load))
        shards[r].append(int(i))
        load[r] += int(keys[i])
    return shards


def kv_head_range(kv_heads: int, world: int, rank: int) -> tuple[int, int]:
    if kv_heads % world:
        raise ValueError(f"{kv_heads} KV heads do not divide over {world} ranks")
    per = kv_heads // world
    return rank * per, (rank + 1) * per


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
