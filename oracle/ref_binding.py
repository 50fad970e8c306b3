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
        if hasattr(L, "ref_prefill_sliding"):
            L.ref_prefill_sliding.restype = c_int
            L.ref_prefill_sliding.argtypes = [_P] * 12 + [c_int] * 4 + [c_float, _P]
            L.ref_prefill_global.restype = c_int
            L.ref_prefill_global.argtypes = [_P] * 11 + [c_int] * 3 + [c_float, _P]
        if hasattr(L, "ref_decode_ingress"):
            L.ref_decode_ingress.restype = c_int
            L.ref_decode_ingress.argtypes = [_P] * 5 + [c_int, _P]
            L.ref_decode_egress.restype = c_int
            L.ref_decode_egress.argtypes = [_P] * 9 + [c_int, _P]
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


def has_prefill() -> bool:
    return available() and hasattr(lib(), "ref_prefill_sliding")


def prefill_sliding(out, q_prepared, k_prepared, v_prepared, q, k, v, q_w, k_w, cos, sin, token_position,
                    batch_size, seqlen_q, seqlen_k, window_size, scale) -> int:
    """The reference's gemma4_flash_attention_sliding_fwd_bf16_norm_rope."""
    return lib().ref_prefill_sliding(_ptr(out), _ptr(q_prepared), _ptr(k_prepared), _ptr(v_prepared), _ptr(q),
                                     _ptr(k), _ptr(v), _ptr(q_w), _ptr(k_w), _ptr(cos), _ptr(sin),
                                     _ptr(token_position), batch_size, seqlen_q, seqlen_k, window_size, scale,
                                     _stream())


def prefill_global(out, q_prepared, k_prepared, v_prepared, q, k, q_w, k_w, cos, sin, token_position, batch_size,
                   seqlen_q, seqlen_k, scale) -> int:
    """The reference's gemma4_flash_attention_global_fwd_bf16_norm_rope."""
    return lib().ref_prefill_global(_ptr(out), _ptr(q_prepared), _ptr(k_prepared), _ptr(v_prepared), _ptr(q),
                                    _ptr(k), _ptr(q_w), _ptr(k_w), _ptr(cos), _ptr(sin), _ptr(token_position),
                                    batch_size, seqlen_q, seqlen_k, scale, _stream())


def has_projections() -> bool:
    return available() and hasattr(lib(), "ref_decode_ingress")


def decode_ingress(raw_qkv, normed_out, x, input_norm_weight, qkv_proj_col_major, global_geometry: bool) -> int:
    """The reference's phase_decode_rmsnorm_project_bf16 (one row), launched cooperatively."""
    return lib().ref_decode_ingress(_ptr(raw_qkv), _ptr(normed_out), _ptr(x), _ptr(input_norm_weight),
                                    _ptr(qkv_proj_col_major), int(global_geometry), _stream())


def decode_egress(residual_out, normed_out, ffn_residual, ffn_x, attention_out, o_proj_col_major, post_norm_weight,
                  pre_ffn_norm_weight, x, global_geometry: bool) -> int:
    """The reference's project_attention_out_post_attention followed by its pre-FFN norm (one row)."""
    return lib().ref_decode_egress(_ptr(residual_out), _ptr(normed_out), _ptr(ffn_residual), _ptr(ffn_x),
                                   _ptr(attention_out), _ptr(o_proj_col_major), _ptr(post_norm_weight),
                                   _ptr(pre_ffn_norm_weight), _ptr(x), int(global_geometry), _stream())
