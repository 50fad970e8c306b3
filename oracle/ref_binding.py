"""ctypes binding of oracle/_ref/libgemma4_ref.so: the reference's own CUDA kernels for the KV path,
compiled for sm_100a by oracle/build_ref.sh. TEST INFRASTRUCTURE ONLY (second checker, golden-vector
source, and the "reference kernels on the same GPU" line of the benchmark). Needs a GPU to run."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int32, c_void_p
from pathlib import Path

from .binding import OrcKvConfig

LIB_PATH = Path(__file__).resolve().parent / "_ref" / "libgemma4_ref.so"
_lib = None
_P = c_void_p


def available() -> bool:
    return LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        L = ctypes.CDLL(str(LIB_PATH))
        L.gemma4_kv_cache_write_bf16.restype = c_int
        L.gemma4_kv_cache_write_bf16.argtypes = [_P, _P, OrcKvConfig, _P, _P, _P, c_int32, c_int32, _P, _P, _P]
        L.ref_decode_append.restype = c_int
        L.ref_decode_append.argtypes = [_P, _P, _P, OrcKvConfig, _P, _P, c_int] + [_P] * 7 + [c_int, _P]
        L.ref_decode_attention.restype = c_int
        L.ref_decode_attention.argtypes = [_P] * 9 + [OrcKvConfig, c_int32, c_float, c_int32, c_int32, c_int32, _P]
        _lib = L
    return _lib


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    import torch

    return torch.cuda.current_stream().cuda_stream


def kv_cache_write(cache_k, cache_v, cfg, page_table, token_batch, token_position, token_count, layer, k, v) -> int:
    return lib().gemma4_kv_cache_write_bf16(_ptr(cache_k), _ptr(cache_v), OrcKvConfig.of(cfg), _ptr(page_table),
                                            _ptr(token_batch), _ptr(token_position), token_count, layer, _ptr(k),
                                            _ptr(v), _stream())


def decode_append(q_prepared, cache_k, cache_v, cfg, page_table, token_position, cache_layer, q, k, v, q_w, k_w,
                  cos, sin, batch_count) -> int:
    return lib().ref_decode_append(_ptr(q_prepared), _ptr(cache_k), _ptr(cache_v), OrcKvConfig.of(cfg),
                                   _ptr(page_table), _ptr(token_position), cache_layer, _ptr(q), _ptr(k), _ptr(v),
                                   _ptr(q_w), _ptr(k_w), _ptr(cos), _ptr(sin), batch_count, _stream())


def decode_attention(out, pm, pl, pacc, q, cache_k, cache_v, page_table, seq_lengths, cfg, layer, scale,
                     split_size, num_splits, batch_count) -> int:
    return lib().ref_decode_attention(_ptr(out), _ptr(pm), _ptr(pl), _ptr(pacc), _ptr(q), _ptr(cache_k),
                                      _ptr(cache_v), _ptr(page_table), _ptr(seq_lengths), OrcKvConfig.of(cfg), layer,
                                      scale, split_size, num_splits, batch_count, _stream())
