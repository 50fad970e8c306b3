"""ctypes binding of the CPU oracle (oracle/kv_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline legs. Product code never imports this module.
All tensors are numpy arrays; bf16 travels as uint16, fp8 e4m3 as uint8.
"""
from __future__ import annotations

import ctypes
import subprocess
from ctypes import POINTER, c_double, c_float, c_int32, c_int64, c_uint16, c_uint8, c_void_p
from pathlib import Path

import numpy as np

ORACLE_DIR = Path(__file__).resolve().parent
LIB_PATH = ORACLE_DIR / "_build" / "libkv_oracle.so"


class OrcKvConfig(ctypes.Structure):
    _fields_ = [(n, c_int32) for n in (
        "num_layers", "num_pages", "page_size", "max_pages_per_seq",
        "batch_size", "num_heads", "head_dim", "window_size")]

    @classmethod
    def of(cls, cfg) -> "OrcKvConfig":
        """From any object with the eight Gemma4KvCacheConfig fields (or a tuple)."""
        if isinstance(cfg, (tuple, list)):
            return cls(*cfg)
        return cls(*(getattr(cfg, n) for n, _ in cls._fields_))

    def cache_elements(self) -> int:
        return (self.num_layers * self.num_pages * self.page_size
                * self.num_heads * self.head_dim)


def build(force: bool = False) -> Path:
    src_newer = (not LIB_PATH.exists()) or any(
        (ORACLE_DIR / f).stat().st_mtime > LIB_PATH.stat().st_mtime
        for f in ("kv_oracle.cpp", "kv_oracle.h"))
    if force or src_newer:
        args = ["make", "-C", str(ORACLE_DIR)] + (["-B"] if force else [])
        proc = subprocess.run(args, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("oracle build failed:\n" + proc.stdout + proc.stderr)
    return LIB_PATH


_lib = None
_P = c_void_p


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        build()
    L = ctypes.CDLL(str(LIB_PATH))
    C = POINTER(OrcKvConfig)
    sigs = {
        "orc_f32_to_bf16": (c_uint16, [c_float]),
        "orc_bf16_to_f32": (c_float, [c_uint16]),
        "orc_f32_to_bf16_n": (None, [_P, _P, c_int64]),
        "orc_bf16_to_f32_n": (None, [_P, _P, c_int64]),
        "orc_f32_to_e4m3": (c_uint8, [c_float]),
        "orc_e4m3_to_f32": (c_float, [c_uint8]),
        "orc_cache_offset": (c_int64, [C] + [c_int32] * 5),
        "orc_make_config": (None, [C, c_int32, c_int32, c_int32, c_int32]),
        "orc_is_global_layer": (c_int32, [c_int32]),
        "orc_layer_index": (c_int32, [c_int32, c_int32]),
        "orc_ensure_page": (c_int32, [_P, _P, C, c_int32, c_int32]),
        "orc_ensure_range": (c_int32, [_P, _P, C, c_int32, c_int32, c_int32]),
        "orc_sliding_pages_per_sequence": (c_int32, [c_int32, c_int32]),
        "orc_runtime_create": (_P, [c_int32, c_int32, c_int32]),
        "orc_runtime_destroy": (None, [_P]),
        "orc_runtime_prepare_prefill": (c_int32, [_P, c_int32]),
        "orc_runtime_prepare_decode_step": (c_int32, [_P]),
        "orc_runtime_array": (c_int64, [_P, c_int32, POINTER(POINTER(c_int32))]),
        "orc_runtime_configs": (None, [_P, C, C, POINTER(c_int32)]),
        "orc_fill_rope_tables": (None, [_P, _P, c_int32, c_int32, c_float, c_int32]),
        "orc_rms_scale": (c_float, [_P, c_int32, c_float]),
        "orc_prep_weighted_rope_head": (None, [_P] * 5 + [c_int32, c_int32]),
        "orc_prep_scale_free_head": (None, [_P, _P, c_int32]),
        "orc_prefill_prep": (None, [_P] * 11 + [c_int64] + [c_int32] * 5),
        "orc_kv_cache_write": (c_int32, [_P, _P, C, _P, _P, _P, c_int32, c_int32, _P, _P]),
        "orc_decode_append": (None, [_P, _P, _P, C, _P, _P, c_int32] + [_P] * 7 + [c_int32] * 4),
        "orc_decode_attention_ref": (None, [_P] * 9 + [C, c_int32, c_float] + [c_int32] * 4),
        "orc_decode_attention_f64": (None, [_P] * 7 + [C, c_int32, c_float, c_int32, c_int32]),
        "orc_fp8_k_index": (c_int64, [C] + [c_int32] * 5),
        "orc_fp8_append": (None, [_P, _P, _P, _P, C, _P, _P, _P, _P, c_int32, c_int32, _P, _P]),
        "orc_fp8_decode_attention_f64": (None, [_P] * 9 + [C, c_int32, c_float, c_int32, c_int32]),
        "orc_prefill_attention_f64": (None, [_P] * 5 + [c_int32] * 6 + [c_float, c_int32]),
        "orc_layer_step_timed": (c_double, [c_int32, _P, _P, _P, _P, C, _P, _P, _P, c_int32] + [_P] * 7 + [c_int32, c_int32, c_float, c_int32]),
        "orc_hardware_threads": (c_int32, []),
        "orc_hidden_rmsnorm": (None, [_P, _P, _P, c_int32]),
        "orc_project_cols": (None, [_P, _P, _P, c_int32, c_int32, c_int32, c_int32]),
        "orc_decode_ingress": (None, [_P] * 5 + [c_int32] * 3),
        "orc_decode_egress": (None, [_P] * 9 + [c_int32] * 3),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def _p(a):
    if a is None:
        return None
    assert isinstance(a, np.ndarray) and a.flags["C_CONTIGUOUS"], "oracle wants contiguous numpy arrays"
    return a.ctypes.data


# ------------------------------------------------------------------ conversions
def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_bf16_n(_p(out), _p(x), x.size)
    return out


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    return (x.astype(np.uint32) << 16).view(np.float32)


def e4m3_to_f32(x: np.ndarray) -> np.ndarray:
    table = np.array([lib().orc_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)
    return table[np.ascontiguousarray(x, dtype=np.uint8)]


# ------------------------------------------------------------------ geometry
def cache_offset(cfg, layer, page, off, head, dim) -> int:
    c = OrcKvConfig.of(cfg)
    return lib().orc_cache_offset(ctypes.byref(c), layer, page, off, head, dim)


def make_config(is_global, num_pages, page_size, max_pages_per_seq) -> OrcKvConfig:
    c = OrcKvConfig()
    lib().orc_make_config(ctypes.byref(c), int(is_global), num_pages, page_size, max_pages_per_seq)
    return c


def ensure_page(page_table, slots, cfg, batch, position) -> int:
    c = OrcKvConfig.of(cfg)
    return lib().orc_ensure_page(_p(page_table), _p(slots), ctypes.byref(c), batch, position)


def ensure_range(page_table, slots, cfg, batch, first, count) -> int:
    c = OrcKvConfig.of(cfg)
    return lib().orc_ensure_range(_p(page_table), _p(slots), ctypes.byref(c), batch, first, count)


def fill_rope_tables(max_seq_len, rotary_half, theta, exponent_dim):
    cos = np.empty((max_seq_len, rotary_half), dtype=np.float32)
    sin = np.empty_like(cos)
    lib().orc_fill_rope_tables(_p(cos), _p(sin), max_seq_len, rotary_half, theta, exponent_dim)
    return cos, sin


class Runtime:
    ARRAYS = {"sliding_page_table": 0, "global_page_table": 1, "sliding_slot_logical_pages": 2,
              "global_slot_logical_pages": 3, "seq_lengths": 4, "token_batch": 5, "token_position": 6}

    def __init__(self, batch_size, max_seq_len, page_size):
        self._h = lib().orc_runtime_create(batch_size, max_seq_len, page_size)
        if not self._h:
            raise ValueError("invalid runtime arguments")

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_runtime_destroy(self._h)
            self._h = None

    def prepare_prefill(self, seq_len) -> int:
        return lib().orc_runtime_prepare_prefill(self._h, seq_len)

    def prepare_decode_step(self) -> int:
        return lib().orc_runtime_prepare_decode_step(self._h)

    def array(self, name) -> np.ndarray:
        ptr = POINTER(c_int32)()
        n = lib().orc_runtime_array(self._h, self.ARRAYS[name], ctypes.byref(ptr))
        if n <= 0:
            return np.zeros(0, dtype=np.int32)
        return np.ctypeslib.as_array(ptr, shape=(n,))

    def configs(self):
        s, g, t = OrcKvConfig(), OrcKvConfig(), c_int32()
        lib().orc_runtime_configs(self._h, ctypes.byref(s), ctypes.byref(g), ctypes.byref(t))
        return s, g, t.value


# ------------------------------------------------------------------ prep / append / write
def prep_weighted_rope_head(x, weight, cos_row, sin_row, rotary_dim):
    out = np.empty_like(x)
    lib().orc_prep_weighted_rope_head(_p(out), _p(x), _p(weight), _p(cos_row), _p(sin_row), x.size, rotary_dim)
    return out


def prep_scale_free_head(x):
    out = np.empty_like(x)
    lib().orc_prep_scale_free_head(_p(out), _p(x), x.size)
    return out


def prefill_prep(q, k, v, q_w, k_w, cos, sin, token_position, q_heads, kv_heads, head_dim, rotary_dim):
    rows = token_position.size
    qp, kp, vp = np.zeros_like(q), np.zeros_like(k), np.zeros_like(k)
    lib().orc_prefill_prep(_p(qp), _p(kp), _p(vp), _p(q), _p(k), _p(v), _p(q_w), _p(k_w), _p(cos), _p(sin),
                           _p(token_position), rows, q_heads, kv_heads, head_dim, rotary_dim, int(v is not None))
    return qp, kp, vp


def kv_cache_write(cache_k, cache_v, cfg, page_table, token_batch, token_position, layer, k, v) -> int:
    c = OrcKvConfig.of(cfg)
    return lib().orc_kv_cache_write(_p(cache_k), _p(cache_v), ctypes.byref(c), _p(page_table), _p(token_batch),
                                    _p(token_position), token_position.size, layer, _p(k), _p(v))


def decode_append(q_prepared, cache_k, cache_v, cfg, page_table, token_position, cache_layer, q, k, v,
                  q_w, k_w, cos, sin, batch_count, q_heads, rotary_dim):
    c = OrcKvConfig.of(cfg)
    lib().orc_decode_append(_p(q_prepared), _p(cache_k), _p(cache_v), ctypes.byref(c), _p(page_table),
                            _p(token_position), cache_layer, _p(q), _p(k), _p(v), _p(q_w), _p(k_w),
                            _p(cos), _p(sin), batch_count, q_heads, rotary_dim, int(v is not None))


# ------------------------------------------------------------------ attention
def decode_attention_ref(q, cache_k, cache_v, page_table, seq_lengths, cfg, layer, scale, split_size,
                         num_splits, batch_count, q_heads, poison=None):
    """Reference-order split + reduce. Returns (out bf16 [B,Hq,D], partial_m, partial_l, partial_acc)."""
    c = OrcKvConfig.of(cfg)
    D = c.head_dim
    out = np.zeros((batch_count, q_heads, D), dtype=np.uint16)
    rows = batch_count * q_heads * num_splits
    fill = np.nan if poison is None else poison
    pm = np.full(rows, fill, dtype=np.float32)
    pl = np.full(rows, fill, dtype=np.float32)
    pacc = np.full(rows * D, fill, dtype=np.float32)
    lib().orc_decode_attention_ref(_p(out), _p(pm), _p(pl), _p(pacc), _p(q), _p(cache_k), _p(cache_v),
                                   _p(page_table), _p(seq_lengths), ctypes.byref(c), layer, scale,
                                   split_size, num_splits, batch_count, q_heads)
    return out, pm, pl, pacc


def decode_attention_f64(q, cache_k, cache_v, page_table, seq_lengths, cfg, layer, scale, batch_count, q_heads):
    c = OrcKvConfig.of(cfg)
    out = np.zeros((batch_count, q_heads, c.head_dim), dtype=np.float32)
    lse = np.zeros((batch_count, q_heads), dtype=np.float32)
    lib().orc_decode_attention_f64(_p(out), _p(lse), _p(q), _p(cache_k), _p(cache_v), _p(page_table),
                                   _p(seq_lengths), ctypes.byref(c), layer, scale, batch_count, q_heads)
    return out, lse


def prefill_attention_f64(q, k, v, batch, seq_len, q_heads, kv_heads, head_dim, window, scale):
    """Causal (+ sliding window) prompt attention in double precision over contiguous prepared rows.
    Returns (out fp32 [batch*seq, q_heads, D], lse fp32 [batch*seq, q_heads])."""
    out = np.empty((batch * seq_len, q_heads, head_dim), dtype=np.float32)
    lse = np.empty((batch * seq_len, q_heads), dtype=np.float32)
    lib().orc_prefill_attention_f64(_p(out), _p(lse), _p(q), _p(k), _p(v), batch, seq_len, q_heads, kv_heads,
                                    head_dim, window, scale, lib().orc_hardware_threads())
    return out, lse


def fp8_k_rows(cache_k, cfg) -> np.ndarray:
    """The fp8 K cache re-ordered to [layer, page, token, head, dim] (undoes the block / swizzle layout)."""
    c = OrcKvConfig.of(cfg)
    tok = np.arange(c.page_size)
    dim = np.arange(c.head_dim)
    head = np.arange(c.num_heads)
    block, tk = tok >> 3, tok & 7
    granule = (dim[None, :] >> 4) ^ ((tk[:, None] & 1) << 2)                        # [token, dim]
    inner = granule * 16 + (dim[None, :] & 15)
    idx = (block[:, None, None] * 8 * c.num_heads * c.head_dim + head[None, :, None] * 8 * c.head_dim
           + tk[:, None, None] * c.head_dim + inner[:, None, :])                      # [token, head, dim]
    pages = np.asarray(cache_k).reshape(c.num_layers, c.num_pages, -1)
    return pages[:, :, idx]


def fp8_append(cache_k, cache_v, scale_k, scale_v, cfg, page_table, seq_batch, first_position, row_count,
               layer, k_prepared, v_prepared):
    c = OrcKvConfig.of(cfg)
    lib().orc_fp8_append(_p(cache_k), _p(cache_v), _p(scale_k), _p(scale_v), ctypes.byref(c), _p(page_table),
                         _p(seq_batch), _p(first_position), _p(row_count), seq_batch.size, layer,
                         _p(k_prepared), _p(v_prepared))


def fp8_decode_attention_f64(q, cache_k, cache_v, scale_k, scale_v, page_table, seq_lengths, cfg, layer,
                             scale, batch_count, q_heads):
    c = OrcKvConfig.of(cfg)
    out = np.zeros((batch_count, q_heads, c.head_dim), dtype=np.float32)
    lse = np.zeros((batch_count, q_heads), dtype=np.float32)
    lib().orc_fp8_decode_attention_f64(_p(out), _p(lse), _p(q), _p(cache_k), _p(cache_v), _p(scale_k),
                                       _p(scale_v), _p(page_table), _p(seq_lengths), ctypes.byref(c), layer,
                                       scale, batch_count, q_heads)
    return out, lse


def layer_step_timed(threads, out, q_prepared, cache_k, cache_v, cfg, page_table, token_position, seq_lengths,
                     cache_layer, q, k, v, q_w, k_w, cos, sin, batch_count, q_heads, scale, split_size) -> float:
    c = OrcKvConfig.of(cfg)
    return lib().orc_layer_step_timed(threads, _p(out), _p(q_prepared), _p(cache_k), _p(cache_v), ctypes.byref(c),
                                      _p(page_table), _p(token_position), _p(seq_lengths), cache_layer, _p(q),
                                      _p(k), _p(v), _p(q_w), _p(k_w), _p(cos), _p(sin), batch_count, q_heads,
                                      scale, split_size)


def hardware_threads() -> int:
    return lib().orc_hardware_threads()


# ------------------------------------------------------------------ decode projections
def hidden_rmsnorm(x, weight):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty_like(x)
    lib().orc_hidden_rmsnorm(_p(out), _p(x), _p(weight), x.size)
    return out


def decode_ingress(x, input_norm_weight, qkv_proj_col_major, threads=0):
    """x [hidden] bf16 bits, weights [cols, hidden]; returns (raw_qkv [cols], normed [hidden])."""
    cols, hidden = qkv_proj_col_major.shape
    raw = np.empty(cols, dtype=np.uint16)
    normed = np.empty(hidden, dtype=np.uint16)
    lib().orc_decode_ingress(_p(raw), _p(normed), _p(x), _p(input_norm_weight), _p(qkv_proj_col_major),
                             hidden, cols, threads or hardware_threads())
    return raw, normed


def decode_egress(attention_out, o_proj_col_major, post_norm_weight, pre_ffn_norm_weight, x, threads=0):
    """attention_out [width], weights [hidden, width]; returns residual_out, normed_out, ffn_residual, ffn_x."""
    hidden, width = o_proj_col_major.shape
    outs = [np.empty(hidden, dtype=np.uint16) for _ in range(4)]
    lib().orc_decode_egress(_p(outs[0]), _p(outs[1]), _p(outs[2]), _p(outs[3]), _p(attention_out),
                            _p(o_proj_col_major), _p(post_norm_weight), _p(pre_ffn_norm_weight), _p(x),
                            width, hidden, threads or hardware_threads())
    return tuple(outs)
