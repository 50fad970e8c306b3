"""ctypes binding of libgemma4_b200kv.so, the B200 implementation of gemma.c's
KV-cache hot path (fused K/V append, paged ring / linear cache, split-KV
flash-decode).

The product is the C-ABI library (``include/gemma4_b200kv.h``) and the C++
host code behind it; this module only loads it and passes raw device pointers
through, so that tests and the benchmark call exactly what a C or C++ caller
would. There is no CPU or PyTorch fallback: if the library is missing or was
not built for sm_100a, loading raises.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path
from typing import Optional

import numpy as np

from . import build as _build

CUDA_SUCCESS = 0
CUDA_ERROR_INVALID_VALUE = 1
NORM_RSQRT_APPROX = 0
NORM_IEEE = 1
STATUS_OK = 0
STATUS_WAIT_TIMEOUT = 1


class KvConfig(ctypes.Structure):
    """Gemma4KvCacheConfig (src/gemma4_kv_cache.cuh:9-18)."""

    _fields_ = [
        ("num_layers", c_int32),
        ("num_pages", c_int32),
        ("page_size", c_int32),
        ("max_pages_per_seq", c_int32),
        ("batch_size", c_int32),
        ("num_heads", c_int32),
        ("head_dim", c_int32),
        ("window_size", c_int32),
    ]

    def astuple(self):
        return tuple(getattr(self, f) for f, _ in self._fields_)

    def cache_elements(self) -> int:
        return (self.num_layers * self.num_pages * self.page_size
                * self.num_heads * self.head_dim)


class RuntimeGeometry(ctypes.Structure):
    _fields_ = [
        ("sliding_layers", c_int32), ("sliding_kv_heads", c_int32),
        ("sliding_head_dim", c_int32), ("sliding_window", c_int32),
        ("sliding_rotary_dim", c_int32), ("sliding_rope_theta", c_float),
        ("global_layers", c_int32), ("global_kv_heads", c_int32),
        ("global_head_dim", c_int32), ("global_rotary_dim", c_int32),
        ("global_rope_theta", c_float), ("global_rope_exponent_dim", c_int32),
    ]


class RuntimeView(ctypes.Structure):
    _fields_ = [
        ("batch_size", c_int32), ("max_seq_len", c_int32),
        ("page_size", c_int32), ("token_count", c_int32),
        ("sliding_cache_config", KvConfig), ("global_cache_config", KvConfig),
        ("sliding_cache_k", c_void_p), ("sliding_cache_v", c_void_p),
        ("global_cache_k", c_void_p), ("global_cache_v", c_void_p),
        ("sliding_page_table", c_void_p), ("global_page_table", c_void_p),
        ("seq_lengths", c_void_p), ("token_batch", c_void_p),
        ("token_position", c_void_p),
        ("sliding_cos", c_void_p), ("sliding_sin", c_void_p),
        ("global_cos", c_void_p), ("global_sin", c_void_p),
        ("h_sliding_page_table", POINTER(c_int32)),
        ("h_global_page_table", POINTER(c_int32)),
        ("h_sliding_slot_logical_pages", POINTER(c_int32)),
        ("h_global_slot_logical_pages", POINTER(c_int32)),
        ("h_seq_lengths", POINTER(c_int32)),
        ("h_token_batch", POINTER(c_int32)),
        ("h_token_position", POINTER(c_int32)),
        ("h_sliding_page_table_size", c_int64),
        ("h_global_page_table_size", c_int64),
        ("h_token_rows", c_int64),
    ]


class LayerStepArgs(ctypes.Structure):
    """B200KvLayerStepArgs: the attention_* fields of
    Gemma4DecodeMegakernelLayerArgs (src/gemma4_megakernel.cuh:42-66)."""

    _fields_ = [
        ("q", c_void_p), ("out", c_void_p), ("lse", c_void_p),
        ("partial_m", c_void_p), ("partial_l", c_void_p),
        ("partial_acc", c_void_p),
        ("cache_k", c_void_p), ("cache_v", c_void_p),
        ("cache_config", KvConfig),
        ("page_table", c_void_p), ("token_position", c_void_p),
        ("seq_lengths", c_void_p),
        ("cache_layer", c_int32), ("split_size", c_int32),
        ("num_splits", c_int32), ("softmax_scale", c_float),
        ("raw_q", c_void_p), ("raw_k", c_void_p), ("raw_v", c_void_p),
        ("q_norm_weight", c_void_p), ("k_norm_weight", c_void_p),
        ("cos", c_void_p), ("sin", c_void_p),
        ("batch_count", c_int32), ("q_heads", c_int32),
        ("rotary_dim", c_int32), ("norm_mode", c_int32),
        ("status", c_void_p),
        ("event_before_attention", c_void_p), ("event_after_attention", c_void_p),
        ("ticket", c_void_p),
        ("peer_gather", c_void_p),
    ]


class IngressArgs(ctypes.Structure):
    """B200KvIngressArgs: input RMSNorm + [Q|K|V] projection
    (src/gemma4_flash_attention_decode.cu:447-496)."""

    _fields_ = [
        ("raw_qkv", c_void_p), ("x", c_void_p), ("input_norm_weight", c_void_p),
        ("qkv_proj_col_major", c_void_p),
        ("batch_count", c_int32), ("hidden_size", c_int32),
        ("cols", c_int32), ("q_width", c_int32), ("k_width", c_int32),
        ("norm_mode", c_int32), ("status", c_void_p),
    ]


class EgressArgs(ctypes.Structure):
    """B200KvEgressArgs: O projection + post-attention norm + residual
    (src/gemma4_flash_attention_decode.cu:35-129)."""

    _fields_ = [
        ("residual_out", c_void_p), ("normed_out", c_void_p), ("ffn_residual", c_void_p),
        ("ffn_x", c_void_p), ("attention_out", c_void_p), ("o_proj_col_major", c_void_p),
        ("post_norm_weight", c_void_p), ("pre_ffn_norm_weight", c_void_p),
        ("x", c_void_p), ("ticket", c_void_p),
        ("batch_count", c_int32), ("hidden_size", c_int32),
        ("attention_width", c_int32), ("norm_mode", c_int32), ("status", c_void_p),
    ]


class AttentionLayerArgs(ctypes.Structure):
    """B200KvAttentionLayerArgs: ingress + layer-step + egress, the attention
    half of Gemma4DecodeMegakernelLayerArgs (src/gemma4_megakernel.cuh:32-66)."""

    _fields_ = [
        ("kv", LayerStepArgs),
        ("attention_x", c_void_p), ("attention_input_norm_weight", c_void_p),
        ("attention_qkv_proj_col_major", c_void_p), ("attention_o_proj_col_major", c_void_p),
        ("attention_post_norm_weight", c_void_p), ("attention_pre_ffn_norm_weight", c_void_p),
        ("raw_qkv", c_void_p),
        ("residual_out", c_void_p), ("normed_out", c_void_p), ("ffn_residual", c_void_p),
        ("ffn_x", c_void_p), ("ticket", c_void_p),
        ("hidden_size", c_int32), ("has_v_projection", c_int32),
    ]


class CudaError(RuntimeError):
    def __init__(self, code: int, where: str):
        super().__init__(f"{where} returned cudaError {code}")
        self.code = code


# Every symbol include/gemma4_b200kv.h declares: name -> (restype, argtypes).
_P = c_void_p
_SIGNATURES = {
    "gemma4_kv_cache_write_bf16": (c_int, [_P, _P, KvConfig, _P, _P, _P, c_int32, c_int32, _P, _P, _P]),
    "b200kv_flash_attention_sliding_fwd_bf16_norm_rope": (c_int, [_P] * 12 + [c_int32] * 4 + [c_float, _P]),
    "b200kv_flash_attention_global_fwd_bf16_norm_rope": (c_int, [_P] * 11 + [c_int32] * 3 + [c_float, _P]),
    "b200kv_prefill_attention_bf16": (c_int, [_P] * 4 + [c_int32] * 6 + [c_float, _P]),
    "b200kv_prefill_attention_fault": (c_int, []),
    "b200kv_prefill_cache_fill_bf16": (c_int, [_P, _P, KvConfig, _P, _P, _P, c_int32, c_int32, c_int32, _P, _P, _P]),
    "b200kv_cache_offset": (c_int64, [POINTER(KvConfig), c_int32, c_int32, c_int32, c_int32, c_int32]),
    "b200kv_make_config": (None, [POINTER(KvConfig), c_int32, c_int32, c_int32, c_int32]),
    "b200kv_is_global_layer": (c_int32, [c_int32]),
    "b200kv_layer_index": (c_int32, [c_int32, c_int32]),
    "b200kv_ensure_page": (c_int32, [_P, _P, POINTER(KvConfig), c_int32, c_int32]),
    "b200kv_ensure_range": (c_int32, [_P, _P, POINTER(KvConfig), c_int32, c_int32, c_int32]),
    "b200kv_sliding_pages_per_sequence": (c_int32, [c_int32, c_int32]),
    "b200kv_fill_rope_tables": (None, [_P, _P, c_int32, c_int32, c_float, c_int32]),
    "b200kv_runtime_geometry_default": (None, [POINTER(RuntimeGeometry)]),
    "b200kv_runtime_state_create": (c_int, [POINTER(_P), c_int32, c_int32, c_int32, POINTER(RuntimeGeometry), _P]),
    "b200kv_runtime_state_destroy": (None, [_P]),
    "b200kv_runtime_prepare_prefill": (c_int, [_P, c_int32, _P]),
    "b200kv_runtime_prepare_decode_step": (c_int, [_P, _P]),
    "b200kv_runtime_state_view": (None, [_P, POINTER(RuntimeView)]),
    "b200kv_prefill_prep_bf16": (c_int, [_P] * 11 + [c_int64, c_int32, c_int32, c_int32, c_int32, c_int32, _P]),
    "b200kv_decode_append_bf16": (c_int, [_P, _P, _P, KvConfig, _P, _P, c_int32] + [_P] * 7 + [c_int32, c_int32, c_int32, c_int32, _P]),
    "b200kv_decode_attention_bf16": (c_int, [_P, _P, _P, _P, _P, KvConfig, _P, _P, c_int32, c_float, c_int32, c_int32, c_int32, c_int32, _P, _P, _P, _P, _P]),
    "b200kv_decode_attention_static_scratch_bf16": (c_int, [_P, _P, _P, _P, _P, KvConfig, _P, _P, c_int32, c_float, c_int32, c_int32, c_int32, c_int32, _P, _P]),
    "b200kv_decode_append_fp8": (c_int, [_P, _P, _P, _P, _P, KvConfig, _P, _P, c_int32] + [_P] * 7 + [c_int32, c_int32, c_int32, c_int32, _P]),
    "b200kv_fp8_append_rows": (c_int, [_P, _P, _P, _P, KvConfig, _P, _P, _P, _P, _P, c_int32, c_int32, c_int32, _P, _P, _P]),
    "b200kv_decode_attention_fp8": (c_int, [_P] * 7 + [KvConfig, _P, _P, c_int32, c_float, c_int32, c_int32, c_int32, _P, _P, _P, _P, _P]),
    "b200kv_decode_workspace_bytes": (None, [c_int32, c_int32, c_int32, c_int32, POINTER(c_size_t), POINTER(c_size_t), POINTER(c_size_t)]),
    "b200kv_plan_splits": (None, [c_int32, c_int32, c_int32, c_int32, POINTER(c_int32), POINTER(c_int32)]),
    "b200kv_plan_balanced": (None, [c_int32, c_int32, POINTER(c_int32)]),
    "b200kv_plan_splits_total": (None, [c_int32, c_int32, c_int64, c_int32, c_int32, POINTER(c_int32), POINTER(c_int32)]),
    "b200kv_decode_layer_step_bf16": (c_int, [POINTER(LayerStepArgs), _P]),
    "b200kv_decode_step_bf16": (c_int, [POINTER(LayerStepArgs), c_int32, _P]),
    "b200kv_decode_step_plan": (c_int, [POINTER(LayerStepArgs), c_int32, POINTER(c_int32), POINTER(c_int32),
                                        POINTER(c_int32)]),
    "b200kv_decode_layer_step_tiled_bf16": (c_int, [POINTER(LayerStepArgs), _P]),
    "b200kv_layer_step_launches": (c_int32, [POINTER(LayerStepArgs)]),
    "b200kv_decode_attention_tiled_bf16": (c_int, [_P, _P, _P, _P, _P, KvConfig, _P, _P, c_int32, c_float, c_int32,
                                                  c_int32, c_int32, _P, _P, _P, _P, _P, _P]),
    "b200kv_decode_ingress_bf16": (c_int, [POINTER(IngressArgs), _P]),
    "b200kv_decode_egress_bf16": (c_int, [POINTER(EgressArgs), _P]),
    "b200kv_decode_attention_layer_bf16": (c_int, [POINTER(AttentionLayerArgs), _P]),
    "b200kv_peer_buffer_create": (c_int, [c_int64, c_int32, c_int32, POINTER(_P), _P]),
    "b200kv_peer_buffer_connect": (c_int, [_P, _P]),
    "b200kv_peer_allgather": (c_int, [_P, _P, c_int64, _P, _P, POINTER(_P)]),
    "b200kv_peer_merge_attention": (c_int, [_P, _P, _P, _P, _P, c_int32, c_int32, _P, _P]),
    "b200kv_peer_buffer_destroy": (c_int, [_P]),
    "b200kv_peer_buffer_set_wait_clocks": (c_int, [_P, c_int64]),
    "b200kv_peer_buffer_reset": (c_int, [_P]),
    "b200kv_peer_buffer_gathered": (c_int, [_P, POINTER(_P)]),
    "b200kv_peer_buffer_create_loopback": (c_int, [c_int64, c_int32, c_int32, POINTER(_P)]),
    "b200kv_peer_buffer_post": (c_int, [_P, c_int32, ctypes.c_uint32, _P]),
    "b200kv_bounded_wait_selftest": (c_int, [c_int64, _P, _P, _P]),
    "b200kv_shard_sequences": (c_int32, [_P, c_int32, c_int32, _P]),
    "b200kv_kv_head_range": (c_int32, [c_int32, c_int32, c_int32, POINTER(c_int32), POINTER(c_int32)]),
    "b200kv_key_range_page_table": (c_int32, [_P, c_int32, c_int32, c_int32, c_int32, c_int32, _P, POINTER(c_int32),
                                             POINTER(c_int32)]),
    "b200kv_timer_create": (c_int, [POINTER(_P)]),
    "b200kv_timer_destroy": (c_int, [_P]),
    "b200kv_timer_record": (c_int, [_P, _P]),
    "b200kv_timer_elapsed_ms": (c_int, [_P, _P, POINTER(c_float)]),
    "b200kv_compiled_arch": (c_int32, []),
}

_lib: Optional[ctypes.CDLL] = None


def library_path() -> Path:
    return _build.LIB_PATH


def load_library(build_if_missing: bool = True) -> ctypes.CDLL:
    """Load the CUDA library; raises if it cannot be found, built or bound."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if build_if_missing and not _build.is_current():
        _build.build()
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with gemma.c_b200/build.py (nvcc, sm_100a); "
            "there is no fallback path")
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if a declared symbol is absent
        fn.restype = restype
        fn.argtypes = argtypes
    if lib.b200kv_compiled_arch() != 1000:
        raise RuntimeError("libgemma4_b200kv.so was not compiled for sm_100a")
    _lib = lib
    return lib


def declared_symbols() -> list[str]:
    return list(_SIGNATURES)


def _ptr(t) -> Optional[int]:
    """Raw address of a torch tensor / numpy array / int / None."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if isinstance(t, np.ndarray):
        return t.ctypes.data
    return t.data_ptr()


def _stream(stream) -> Optional[int]:
    if stream is None:
        import torch

        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


def _check(code: int, where: str, check: bool) -> int:
    if check and code != CUDA_SUCCESS:
        raise CudaError(code, where)
    return code


def make_kv_config(num_layers, num_pages, page_size, max_pages_per_seq,
                   batch_size, num_heads, head_dim, window_size) -> KvConfig:
    return KvConfig(num_layers, num_pages, page_size, max_pages_per_seq,
                    batch_size, num_heads, head_dim, window_size)


# ---------------------------------------------------------------- host helpers
def cache_offset(cfg: KvConfig, layer, page, page_offset, head, dim) -> int:
    return load_library().b200kv_cache_offset(ctypes.byref(cfg), layer, page, page_offset, head, dim)


def make_config(is_global: bool, num_pages: int, page_size: int, max_pages_per_seq: int) -> KvConfig:
    cfg = KvConfig()
    load_library().b200kv_make_config(ctypes.byref(cfg), int(is_global), num_pages, page_size, max_pages_per_seq)
    return cfg


def is_global_layer(layer: int) -> bool:
    return bool(load_library().b200kv_is_global_layer(layer))


def layer_index(model_layer: int, global_cache: bool) -> int:
    return load_library().b200kv_layer_index(model_layer, int(global_cache))


def ensure_page(page_table: np.ndarray, slot_logical_pages: np.ndarray, cfg: KvConfig, batch: int, position: int) -> int:
    return load_library().b200kv_ensure_page(_ptr(page_table), _ptr(slot_logical_pages), ctypes.byref(cfg), batch, position)


def ensure_range(page_table: np.ndarray, slot_logical_pages: np.ndarray, cfg: KvConfig, batch: int, first_position: int, token_count: int) -> int:
    return load_library().b200kv_ensure_range(_ptr(page_table), _ptr(slot_logical_pages), ctypes.byref(cfg), batch, first_position, token_count)


def sliding_pages_per_sequence(max_seq_len: int, page_size: int) -> int:
    return load_library().b200kv_sliding_pages_per_sequence(max_seq_len, page_size)


def fill_rope_tables(max_seq_len: int, rotary_half: int, theta: float, exponent_dim: int):
    cos = np.empty((max_seq_len, rotary_half), dtype=np.float32)
    sin = np.empty_like(cos)
    load_library().b200kv_fill_rope_tables(_ptr(cos), _ptr(sin), max_seq_len, rotary_half, theta, exponent_dim)
    return cos, sin


def plan_splits(batch_count: int, max_live_keys: int, kv_heads: int, sm_count: int):
    size, count = c_int32(), c_int32()
    load_library().b200kv_plan_splits(batch_count, max_live_keys, kv_heads, sm_count, ctypes.byref(size), ctypes.byref(count))
    return size.value, count.value


def plan_balanced(batch_count: int, sm_count: int) -> int:
    """num_splits to pass with split_size == 0 (balanced partition)."""
    n = c_int32()
    load_library().b200kv_plan_balanced(batch_count, sm_count, ctypes.byref(n))
    return n.value


def plan_splits_total(batch_count: int, max_live_keys: int, total_live_keys: int, kv_heads: int, sm_count: int):
    size, count = c_int32(), c_int32()
    load_library().b200kv_plan_splits_total(batch_count, max_live_keys, total_live_keys, kv_heads, sm_count,
                                            ctypes.byref(size), ctypes.byref(count))
    return size.value, count.value


def decode_workspace_bytes(batch_count: int, q_heads: int, head_dim: int, num_splits: int):
    m, l, acc = c_size_t(), c_size_t(), c_size_t()
    load_library().b200kv_decode_workspace_bytes(batch_count, q_heads, head_dim, num_splits, ctypes.byref(m), ctypes.byref(l), ctypes.byref(acc))
    return m.value, l.value, acc.value


def default_geometry() -> RuntimeGeometry:
    g = RuntimeGeometry()
    load_library().b200kv_runtime_geometry_default(ctypes.byref(g))
    return g


class RuntimeState:
    """Handle on a Gemma4RuntimeState (src/gemma4_runtime.cuh:12-64)."""

    def __init__(self, batch_size: int, max_seq_len: int, page_size: int,
                 geometry: Optional[RuntimeGeometry] = None, stream=None, check: bool = True):
        self._lib = load_library()
        self._handle = c_void_p()
        geo = ctypes.byref(geometry) if geometry is not None else None
        self.status = self._lib.b200kv_runtime_state_create(
            ctypes.byref(self._handle), batch_size, max_seq_len, page_size, geo, _stream(stream))
        _check(self.status, "b200kv_runtime_state_create", check)

    def close(self):
        if self._handle:
            self._lib.b200kv_runtime_state_destroy(self._handle)
            self._handle = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def prepare_prefill(self, seq_len: int, stream=None, check: bool = True) -> int:
        return _check(self._lib.b200kv_runtime_prepare_prefill(self._handle, seq_len, _stream(stream)),
                      "b200kv_runtime_prepare_prefill", check)

    def prepare_decode_step(self, stream=None, check: bool = True) -> int:
        return _check(self._lib.b200kv_runtime_prepare_decode_step(self._handle, _stream(stream)),
                      "b200kv_runtime_prepare_decode_step", check)

    def view(self) -> RuntimeView:
        v = RuntimeView()
        self._lib.b200kv_runtime_state_view(self._handle, ctypes.byref(v))
        return v

    def host_array(self, name: str) -> np.ndarray:
        """Writable numpy view of one host mirror (h_seq_lengths, ...)."""
        v = self.view()
        sizes = {
            "h_sliding_page_table": v.h_sliding_page_table_size,
            "h_global_page_table": v.h_global_page_table_size,
            "h_sliding_slot_logical_pages": v.h_sliding_page_table_size,
            "h_global_slot_logical_pages": v.h_global_page_table_size,
            "h_seq_lengths": v.batch_size,
            "h_token_batch": v.h_token_rows,
            "h_token_position": v.h_token_rows,
        }
        n = int(sizes[name])
        if n == 0:
            return np.zeros(0, dtype=np.int32)
        return np.ctypeslib.as_array(getattr(v, name), shape=(n,))


# -------------------------------------------------------------- device entry points
def kv_cache_write(cache_k, cache_v, cfg: KvConfig, page_table, token_batch, token_position,
                   token_count: int, layer: int, k, v, stream=None, check: bool = True) -> int:
    code = load_library().gemma4_kv_cache_write_bf16(
        _ptr(cache_k), _ptr(cache_v), cfg, _ptr(page_table), _ptr(token_batch), _ptr(token_position),
        token_count, layer, _ptr(k), _ptr(v), _stream(stream))
    return _check(code, "gemma4_kv_cache_write_bf16", check)


def flash_attention_sliding_fwd(out, q_prepared, k_prepared, v_prepared, q, k, v, q_norm_weight, k_norm_weight,
                                cos, sin, token_position, batch_size: int, seqlen_q: int, seqlen_k: int,
                                window_size: int, softmax_scale: float, stream=None, check: bool = True) -> int:
    """gemma4_flash_attention_sliding_fwd_bf16_norm_rope: prompt prep + causal sliding-window attention."""
    code = load_library().b200kv_flash_attention_sliding_fwd_bf16_norm_rope(
        _ptr(out), _ptr(q_prepared), _ptr(k_prepared), _ptr(v_prepared), _ptr(q), _ptr(k), _ptr(v),
        _ptr(q_norm_weight), _ptr(k_norm_weight), _ptr(cos), _ptr(sin), _ptr(token_position), batch_size,
        seqlen_q, seqlen_k, window_size, softmax_scale, _stream(stream))
    return _check(code, "b200kv_flash_attention_sliding_fwd_bf16_norm_rope", check)


def flash_attention_global_fwd(out, q_prepared, k_prepared, v_prepared, q, k, q_norm_weight, k_norm_weight,
                               cos, sin, token_position, batch_size: int, seqlen_q: int, seqlen_k: int,
                               softmax_scale: float, stream=None, check: bool = True) -> int:
    """gemma4_flash_attention_global_fwd_bf16_norm_rope: 16 Q / 1 KV x 512, rotary 128, V from raw K."""
    code = load_library().b200kv_flash_attention_global_fwd_bf16_norm_rope(
        _ptr(out), _ptr(q_prepared), _ptr(k_prepared), _ptr(v_prepared), _ptr(q), _ptr(k), _ptr(q_norm_weight),
        _ptr(k_norm_weight), _ptr(cos), _ptr(sin), _ptr(token_position), batch_size, seqlen_q, seqlen_k,
        softmax_scale, _stream(stream))
    return _check(code, "b200kv_flash_attention_global_fwd_bf16_norm_rope", check)


def prefill_attention(out, q_prepared, k_prepared, v_prepared, batch_size: int, seq_len: int, q_heads: int,
                      kv_heads: int, head_dim: int, window_size: int, softmax_scale: float, stream=None,
                      check: bool = True) -> int:
    """Causal (+ window) attention of each sequence over its own prepared rows."""
    code = load_library().b200kv_prefill_attention_bf16(
        _ptr(out), _ptr(q_prepared), _ptr(k_prepared), _ptr(v_prepared), batch_size, seq_len, q_heads, kv_heads,
        head_dim, window_size, softmax_scale, _stream(stream))
    return _check(code, "b200kv_prefill_attention_bf16", check)


def prefill_attention_fault() -> int:
    """Synchronises; 0, or which bounded wait of the head_dim-256 tensor-core kernel ran out last launch."""
    return int(load_library().b200kv_prefill_attention_fault())


def prefill_cache_fill(cache_k, cache_v, cfg: KvConfig, page_table, token_batch, token_position,
                       batch_size: int, seq_len: int, layer: int, k_prepared, v_prepared, stream=None,
                       check: bool = True) -> int:
    """Prompt rows into the cache in one launch; a sliding cache keeps only each sequence's last window."""
    code = load_library().b200kv_prefill_cache_fill_bf16(
        _ptr(cache_k), _ptr(cache_v), cfg, _ptr(page_table), _ptr(token_batch), _ptr(token_position),
        batch_size, seq_len, layer, _ptr(k_prepared), _ptr(v_prepared), _stream(stream))
    return _check(code, "b200kv_prefill_cache_fill_bf16", check)


def prefill_prep(q_prepared, k_prepared, v_prepared, q, k, v, q_norm_weight, k_norm_weight, cos, sin,
                 token_position, rows: int, q_heads: int, kv_heads: int, head_dim: int, rotary_dim: int,
                 norm_mode: int = NORM_RSQRT_APPROX, stream=None, check: bool = True) -> int:
    code = load_library().b200kv_prefill_prep_bf16(
        _ptr(q_prepared), _ptr(k_prepared), _ptr(v_prepared), _ptr(q), _ptr(k), _ptr(v),
        _ptr(q_norm_weight), _ptr(k_norm_weight), _ptr(cos), _ptr(sin), _ptr(token_position),
        rows, q_heads, kv_heads, head_dim, rotary_dim, norm_mode, _stream(stream))
    return _check(code, "b200kv_prefill_prep_bf16", check)


def decode_append(q_prepared, cache_k, cache_v, cfg: KvConfig, page_table, token_position, cache_layer: int,
                  q, k, v, q_norm_weight, k_norm_weight, cos, sin, batch_count: int, q_heads: int,
                  rotary_dim: int, norm_mode: int = NORM_RSQRT_APPROX, stream=None, check: bool = True) -> int:
    code = load_library().b200kv_decode_append_bf16(
        _ptr(q_prepared), _ptr(cache_k), _ptr(cache_v), cfg, _ptr(page_table), _ptr(token_position),
        cache_layer, _ptr(q), _ptr(k), _ptr(v), _ptr(q_norm_weight), _ptr(k_norm_weight), _ptr(cos), _ptr(sin),
        batch_count, q_heads, rotary_dim, norm_mode, _stream(stream))
    return _check(code, "b200kv_decode_append_bf16", check)


def decode_attention(out, lse, q_prepared, cache_k, cache_v, cfg: KvConfig, page_table, seq_lengths,
                     cache_layer: int, softmax_scale: float, split_size: int, num_splits: int,
                     batch_count: int, q_heads: int, partial_m=None, partial_l=None, partial_acc=None,
                     status=None, stream=None, check: bool = True) -> int:
    code = load_library().b200kv_decode_attention_bf16(
        _ptr(out), _ptr(lse), _ptr(q_prepared), _ptr(cache_k), _ptr(cache_v), cfg, _ptr(page_table),
        _ptr(seq_lengths), cache_layer, softmax_scale, split_size, num_splits, batch_count, q_heads,
        _ptr(partial_m), _ptr(partial_l), _ptr(partial_acc), _ptr(status), _stream(stream))
    return _check(code, "b200kv_decode_attention_bf16", check)


STATIC_SCRATCH_BYTES = 16 << 20
TICKETS_PER_HEAD = 11            # B200KV_TICKETS_PER_HEAD: words of LayerStepArgs.ticket per sequence and KV head


def decode_attention_static_scratch(out, lse, q_prepared, cache_k, cache_v, cfg: KvConfig, page_table, seq_lengths,
                                    cache_layer: int, softmax_scale: float, split_size: int, num_splits: int,
                                    batch_count: int, q_heads: int, status=None, stream=None,
                                    check: bool = True) -> int:
    """Decode attention whose split partials live in the library's built-in 16 MiB array: for callers
    that cannot allocate scratch (no allocator of their own, all device memory already committed, or a
    path that must not synchronise the device). Calls on one device share the array; keep them on one stream."""
    code = load_library().b200kv_decode_attention_static_scratch_bf16(
        _ptr(out), _ptr(lse), _ptr(q_prepared), _ptr(cache_k), _ptr(cache_v), cfg, _ptr(page_table),
        _ptr(seq_lengths), cache_layer, softmax_scale, split_size, num_splits, batch_count, q_heads,
        _ptr(status), _stream(stream))
    return _check(code, "b200kv_decode_attention_static_scratch_bf16", check)


def decode_layer_step(args: LayerStepArgs, stream=None, check: bool = True) -> int:
    code = load_library().b200kv_decode_layer_step_bf16(ctypes.byref(args), _stream(stream))
    return _check(code, "b200kv_decode_layer_step_bf16", check)


def layer_step_launches(args: LayerStepArgs) -> int:
    return load_library().b200kv_layer_step_launches(ctypes.byref(args))


def decode_layer_step_tiled(args: LayerStepArgs, stream=None, check: bool = True) -> int:
    """The layer-step as one launch of the per-(sequence, KV head, key range) kernel; needs args.ticket."""
    code = load_library().b200kv_decode_layer_step_tiled_bf16(ctypes.byref(args), _stream(stream))
    return _check(code, "b200kv_decode_layer_step_tiled_bf16", check)


def decode_attention_tiled(out, lse, q_prepared, cache_k, cache_v, cfg: KvConfig, page_table, seq_lengths,
                           cache_layer: int, softmax_scale: float, num_splits: int, batch_count: int, q_heads: int,
                           partial_m, partial_l, partial_acc, ticket, status=None, stream=None,
                           check: bool = True) -> int:
    code = load_library().b200kv_decode_attention_tiled_bf16(
        _ptr(out), _ptr(lse), _ptr(q_prepared), _ptr(cache_k), _ptr(cache_v), cfg, _ptr(page_table),
        _ptr(seq_lengths), cache_layer, softmax_scale, num_splits, batch_count, q_heads, _ptr(partial_m),
        _ptr(partial_l), _ptr(partial_acc), _ptr(ticket), _ptr(status), _stream(stream))
    return _check(code, "b200kv_decode_attention_tiled_bf16", check)


def decode_step(layers, layer_count: int, stream=None, check: bool = True) -> int:
    """`layers` is a ctypes array (LayerStepArgs * n)."""
    code = load_library().b200kv_decode_step_bf16(layers, layer_count, _stream(stream))
    return _check(code, "b200kv_decode_step_bf16", check)


def decode_step_plan(layers, layer_count: int, forwarded: bool = False):
    """What decode_step would tell each entry's launch (host only): per entry the number of unfinished launches
    taken to be earlier steps of its own cache layer, and whether its kernel releases the next entry's at once;
    with `forwarded` also for how many of those steps the kernel prepares the appended rows itself."""
    held = (c_int32 * max(layer_count, 1))()
    early = (c_int32 * max(layer_count, 1))()
    fwd = (c_int32 * max(layer_count, 1))()
    _check(load_library().b200kv_decode_step_plan(layers, layer_count, held, early, fwd), "b200kv_decode_step_plan",
           True)
    out = (list(held)[:layer_count], [bool(x) for x in list(early)[:layer_count]])
    return out + (list(fwd)[:layer_count],) if forwarded else out


def decode_ingress(args: IngressArgs, stream=None, check: bool = True) -> int:
    code = load_library().b200kv_decode_ingress_bf16(ctypes.byref(args), _stream(stream))
    return _check(code, "b200kv_decode_ingress_bf16", check)


def decode_egress(args: EgressArgs, stream=None, check: bool = True) -> int:
    code = load_library().b200kv_decode_egress_bf16(ctypes.byref(args), _stream(stream))
    return _check(code, "b200kv_decode_egress_bf16", check)


def decode_attention_layer(args: AttentionLayerArgs, stream=None, check: bool = True) -> int:
    code = load_library().b200kv_decode_attention_layer_bf16(ctypes.byref(args), _stream(stream))
    return _check(code, "b200kv_decode_attention_layer_bf16", check)


class PeerBuffer:
    """This rank's side of the peer-memory all-gather (b200kv_peer_*): `export` is the 64 bytes the other
    ranks need; connect() takes all ranks' exports in rank order (bytes of length 64 * world)."""

    def __init__(self, slot_bytes: int, world: int, rank: int, loopback: bool = False):
        self.world, self.rank, self.slot_bytes = world, rank, slot_bytes
        self._handle = c_void_p()
        if loopback:       # one-GPU stand-in: the peers are local buffers nobody writes (b200kv_peer_buffer_post)
            _check(load_library().b200kv_peer_buffer_create_loopback(slot_bytes, world, rank, ctypes.byref(self._handle)),
                   "b200kv_peer_buffer_create_loopback", True)
            self.export = b""
            return
        buf = ctypes.create_string_buffer(64)
        _check(load_library().b200kv_peer_buffer_create(slot_bytes, world, rank, ctypes.byref(self._handle), buf),
               "b200kv_peer_buffer_create", True)
        self.export = bytes(buf.raw)

    def set_wait_clocks(self, clocks: int):
        _check(load_library().b200kv_peer_buffer_set_wait_clocks(self._handle, clocks),
               "b200kv_peer_buffer_set_wait_clocks", True)

    def post(self, from_rank: int, epoch: int, stream=None):
        _check(load_library().b200kv_peer_buffer_post(self._handle, from_rank, epoch, _stream(stream)),
               "b200kv_peer_buffer_post", True)

    @property
    def handle(self) -> int:
        """The raw handle, for LayerStepArgs.peer_gather."""
        return self._handle.value

    def gathered(self) -> int:
        """Device address of what the most recent gather delivered ([world][slot_bytes])."""
        out = c_void_p()
        _check(load_library().b200kv_peer_buffer_gathered(self._handle, ctypes.byref(out)),
               "b200kv_peer_buffer_gathered", True)
        return out.value or 0

    def reset(self):
        _check(load_library().b200kv_peer_buffer_reset(self._handle), "b200kv_peer_buffer_reset", True)

    def connect(self, exports: bytes):
        assert len(exports) == 64 * self.world
        _check(load_library().b200kv_peer_buffer_connect(self._handle, exports), "b200kv_peer_buffer_connect", True)

    def allgather(self, src, nbytes: int, status=None, stream=None, check: bool = True) -> int:
        """Enqueue the gather; returns the device address of the [world][slot_bytes] result."""
        out = c_void_p()
        code = load_library().b200kv_peer_allgather(self._handle, _ptr(src), nbytes, _ptr(status), _stream(stream),
                                                    ctypes.byref(out))
        _check(code, "b200kv_peer_allgather", check)
        return out.value or 0

    def merge_attention(self, merged_out, merged_lse, out, lse, rows: int, head_dim: int, status=None, stream=None,
                        check: bool = True) -> int:
        code = load_library().b200kv_peer_merge_attention(self._handle, _ptr(merged_out), _ptr(merged_lse), _ptr(out),
                                                          _ptr(lse), rows, head_dim, _ptr(status), _stream(stream))
        return _check(code, "b200kv_peer_merge_attention", check)

    def close(self):
        if self._handle:
            load_library().b200kv_peer_buffer_destroy(self._handle)
            self._handle = c_void_p()


def bounded_wait_selftest(clock_limit: int, status, waited_clocks=None, stream=None, check: bool = True) -> int:
    code = load_library().b200kv_bounded_wait_selftest(clock_limit, _ptr(status), _ptr(waited_clocks), _stream(stream))
    return _check(code, "b200kv_bounded_wait_selftest", check)


class Timer:
    """A CUDA event owned by the library (for the LayerStepArgs profiling hooks)."""

    def __init__(self):
        self.handle = c_void_p()
        _check(load_library().b200kv_timer_create(ctypes.byref(self.handle)), "b200kv_timer_create", True)

    def record(self, stream=None):
        _check(load_library().b200kv_timer_record(self.handle, _stream(stream)), "b200kv_timer_record", True)

    def elapsed_ms(self, end: "Timer") -> float:
        ms = c_float()
        _check(load_library().b200kv_timer_elapsed_ms(self.handle, end.handle, ctypes.byref(ms)),
               "b200kv_timer_elapsed_ms", True)
        return ms.value

    def close(self):
        if self.handle:
            load_library().b200kv_timer_destroy(self.handle)
            self.handle = c_void_p()


# ------------------------------------------------------------------ fp8 e4m3 cache
def decode_append_fp8(q_prepared, cache_k, cache_v, scale_k, scale_v, cfg: KvConfig, page_table, token_position,
                      cache_layer: int, q, k, v, q_norm_weight, k_norm_weight, cos, sin, batch_count: int,
                      q_heads: int, rotary_dim: int, norm_mode: int = NORM_RSQRT_APPROX, stream=None,
                      check: bool = True) -> int:
    code = load_library().b200kv_decode_append_fp8(
        _ptr(q_prepared), _ptr(cache_k), _ptr(cache_v), _ptr(scale_k), _ptr(scale_v), cfg, _ptr(page_table),
        _ptr(token_position), cache_layer, _ptr(q), _ptr(k), _ptr(v), _ptr(q_norm_weight), _ptr(k_norm_weight),
        _ptr(cos), _ptr(sin), batch_count, q_heads, rotary_dim, norm_mode, _stream(stream))
    return _check(code, "b200kv_decode_append_fp8", check)


def fp8_append_rows(cache_k, cache_v, scale_k, scale_v, cfg: KvConfig, page_table, seq_batch, first_position,
                    row_count, row_start, run_count: int, max_row_count: int, cache_layer: int, k_prepared,
                    v_prepared, stream=None, check: bool = True) -> int:
    code = load_library().b200kv_fp8_append_rows(
        _ptr(cache_k), _ptr(cache_v), _ptr(scale_k), _ptr(scale_v), cfg, _ptr(page_table), _ptr(seq_batch),
        _ptr(first_position), _ptr(row_count), _ptr(row_start), run_count, max_row_count, cache_layer,
        _ptr(k_prepared), _ptr(v_prepared), _stream(stream))
    return _check(code, "b200kv_fp8_append_rows", check)


def decode_attention_fp8(out, lse, q_prepared, cache_k, cache_v, scale_k, scale_v, cfg: KvConfig, page_table,
                         seq_lengths, cache_layer: int, softmax_scale: float, num_splits: int, batch_count: int,
                         q_heads: int, partial_m, partial_l, partial_acc, status=None, stream=None,
                         check: bool = True) -> int:
    code = load_library().b200kv_decode_attention_fp8(
        _ptr(out), _ptr(lse), _ptr(q_prepared), _ptr(cache_k), _ptr(cache_v), _ptr(scale_k), _ptr(scale_v), cfg,
        _ptr(page_table), _ptr(seq_lengths), cache_layer, softmax_scale, num_splits, batch_count, q_heads,
        _ptr(partial_m), _ptr(partial_l), _ptr(partial_acc), _ptr(status), _stream(stream))
    return _check(code, "b200kv_decode_attention_fp8", check)
