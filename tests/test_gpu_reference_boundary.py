"""The drop-in boundary proved with the reference's own programs.

oracle/build_ref.sh compiles, where the gemma.c sources are mounted, (a) the reference's unchanged
tests/test_kv_cache.cu, tests/test_runtime_state.cu and tests/test_flash_attention.cu against the library's stand-in
headers (include/compat) and links them to libgemma4_b200kv.so alone, and (b) tests/cpp/megakernel_layer.cu, which
includes the reference's real gemma4_megakernel.cuh / gemma4_runtime.cuh and drives one decode layer with the
reference's own Gemma4RuntimeState and Gemma4DecodeMegakernelLayerArgs. The executables travel with the tree
(oracle/_ref/); here they run on the GPU. Without them (a checkout that never saw the gemma.c sources) the tests skip.
"""
from __future__ import annotations

import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.gpu_util import dev, host_u16
from tests.helpers import ATTN_MAX_ABS, ATTN_MAX_REL, attention_error

pytestmark = pytest.mark.gpu

REF_DIR = Path(__file__).resolve().parent.parent / "oracle" / "_ref"


def _exe(name: str) -> Path:
    path = REF_DIR / name
    if not path.is_file():
        pytest.skip(f"oracle/_ref/{name} not built (needs the gemma.c sources at build time)")
    return path


@pytest.mark.parametrize("name,banner", [
    ("ref_test_kv_cache", "kv cache tests passed"),                  # tests/test_kv_cache.cu:94-140
    ("ref_test_runtime_state", "runtime state tests passed"),        # tests/test_runtime_state.cu:29-150
    ("ref_test_flash_attention", "flash attention tests passed"),    # tests/test_flash_attention.cu:175-354
])
def test_reference_test_program_passes_against_the_library(kv, name, banner):
    """The reference's own test executable, built from its unchanged source against the library, prints its
    pass line and exits 0."""
    kv.load_library(build_if_missing=False)
    run = subprocess.run([str(_exe(name))], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    assert banner in run.stdout


def test_decode_layer_through_the_reference_structs(kv, orc, tmp_path):
    """A decode layer driven from C++ with the reference's Gemma4RuntimeState (initialised, advanced and freed by
    the library) and its Gemma4DecodeMegakernelLayerArgs, three steps after a 1500-token prompt on sliding layer 0.
    Checked: the struct size the program saw is the reference's; the raw projection rows, prepared q, cache and
    the four layer outputs are the bits the same call gives through the C ABI (ctypes) on the same inputs; the
    attention rows are within the bf16 band of the double-precision oracle over the cache the program left."""
    exe = _exe("megakernel_layer")
    HID, HQ, H, D = 3840, 16, 8, 256
    q_width, k_width, cols = HQ * D, H * D, HQ * D + 2 * H * D
    rng = np.random.default_rng(2027)
    bits = lambda a: orc.f32_to_bf16(a.astype(np.float32))
    inp = {
        "x": bits(rng.standard_normal(HID)),
        "w_in": bits(1.0 + 0.05 * rng.standard_normal(HID)),
        "w_qkv": bits(rng.standard_normal((cols, HID)) * HID ** -0.5),
        "w_o": bits(rng.standard_normal((HID, q_width)) * q_width ** -0.5),
        "w_post": bits(1.0 + 0.05 * rng.standard_normal(HID)),
        "w_pre": bits(1.0 + 0.05 * rng.standard_normal(HID)),
        "q_w": bits(1.0 + 0.05 * rng.standard_normal(D)),
        "k_w": bits(1.0 + 0.05 * rng.standard_normal(D)),
    }
    for name, a in inp.items():
        a.tofile(tmp_path / f"{name}.bin")
    prompt, steps = 1500, 3
    run = subprocess.run([str(exe), str(tmp_path), str(prompt), str(steps)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    meta = (tmp_path / "meta.txt").read_text().split()
    cfg_t = tuple(int(v) for v in meta[:8])
    seq_len, position, num_splits, status, state_size = (int(v) for v in meta[8:13])
    assert status == 0 and seq_len == prompt + steps and position == prompt + steps - 1
    assert state_size == 184 + 7 * 24                      # src/gemma4_runtime.cuh:12-42 on an LP64 host
    assert cfg_t[2:] == (16, 65, 1, 8, 256, 1024)          # page 16, ring of 65 pages (src/gemma4_runtime.cu:18-24)

    load = lambda n, dt=np.uint16: np.fromfile(tmp_path / f"{n}.bin", dtype=dt)
    table = load("page_table", np.int32).reshape(1, -1)
    cos = load("cos", np.float32).reshape(-1, D // 2)
    sin = load("sin", np.float32).reshape(-1, D // 2)
    ck_after, cv_after = load("cache_k"), load("cache_v")
    one_layer = (1,) + cfg_t[1:]

    # the same last step through the C ABI, starting from the cache as the program left it (the new row is
    # rewritten with the same bits)
    cfg = kv.make_kv_config(*one_layer)
    d = {n: dev(v) for n, v in inp.items()}
    d.update(ck=dev(ck_after), cv=dev(cv_after), table=dev(table), cos=dev(cos), sin=dev(sin),
             pos=dev(np.array([position], np.int32)), length=dev(np.array([seq_len], np.int32)))
    q = torch.zeros(q_width, dtype=torch.int16, device="cuda")
    out, raw = torch.zeros_like(q), torch.zeros(8704, dtype=torch.int16, device="cuda")
    outs = [torch.zeros(HID, dtype=torch.int16, device="cuda") for _ in range(4)]
    pm = torch.zeros(HQ * num_splits, dtype=torch.float32, device="cuda")
    pl, pacc = pm.clone(), torch.zeros(HQ * num_splits * D, dtype=torch.float32, device="cuda")
    # one word for the O projection's row, then the attention's tickets: the layout the C++ entry point hands
    # on (include/gemma4_b200kv.hpp), so that both runs take the one-launch attention kernel
    ticket = torch.zeros(1 + 8 * kv.TICKETS_PER_HEAD, dtype=torch.int32, device="cuda")
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    a = kv.AttentionLayerArgs()
    s = a.kv
    s.q, s.out, s.lse = q.data_ptr(), out.data_ptr(), None
    s.partial_m, s.partial_l, s.partial_acc = pm.data_ptr(), pl.data_ptr(), pacc.data_ptr()
    s.cache_k, s.cache_v, s.cache_config = d["ck"].data_ptr(), d["cv"].data_ptr(), cfg
    s.page_table, s.token_position, s.seq_lengths = d["table"].data_ptr(), d["pos"].data_ptr(), d["length"].data_ptr()
    s.cache_layer, s.split_size, s.num_splits, s.softmax_scale = 0, 0, num_splits, 1.0 / 16.0
    s.q_norm_weight, s.k_norm_weight, s.cos, s.sin = (d["q_w"].data_ptr(), d["k_w"].data_ptr(), d["cos"].data_ptr(),
                                                     d["sin"].data_ptr())
    s.batch_count, s.q_heads, s.rotary_dim, s.norm_mode, s.status = 1, HQ, D, kv.NORM_RSQRT_APPROX, st.data_ptr()
    s.ticket = ticket.data_ptr() + 4
    a.attention_x, a.attention_input_norm_weight = d["x"].data_ptr(), d["w_in"].data_ptr()
    a.attention_qkv_proj_col_major, a.attention_o_proj_col_major = d["w_qkv"].data_ptr(), d["w_o"].data_ptr()
    a.attention_post_norm_weight, a.attention_pre_ffn_norm_weight = d["w_post"].data_ptr(), d["w_pre"].data_ptr()
    a.raw_qkv = raw.data_ptr()
    a.residual_out, a.normed_out, a.ffn_residual, a.ffn_x = (t.data_ptr() for t in outs)
    a.ticket, a.hidden_size, a.has_v_projection = ticket.data_ptr(), HID, 1
    kv.decode_attention_layer(a)
    torch.cuda.synchronize()
    assert st[0].item() == 0
    assert np.array_equal(host_u16(raw)[:cols], load("raw"))
    assert np.array_equal(host_u16(q), load("q"))
    assert np.array_equal(host_u16(d["ck"]), ck_after) and np.array_equal(host_u16(d["cv"]), cv_after)
    for name, t in zip(("residual_out", "normed_out", "ffn_residual", "ffn_x"), outs):
        got, want = load(name), host_u16(t)
        assert np.array_equal(got, want), (name, int((got != want).sum()))
    assert np.array_equal(load("attn"), host_u16(out))

    # the appended rows sit where the reference's addressing puts them and the attention is the oracle's
    for p in range(prompt, prompt + steps):
        slot = (p // 16) % cfg_t[3]
        row = (int(table[0, slot]) * 16 + p % 16) * H * D
        pattern = ((np.arange(row, row + H * D, dtype=np.int64) * 37 + 17) % 257 - 128) / 64.0
        assert not np.array_equal(ck_after[row:row + H * D], bits(pattern)), f"position {p} was not appended"
    ref, _ = orc.decode_attention_f64(load("q").reshape(1, HQ, D), ck_after, cv_after, table,
                                      np.array([seq_len], np.int32), one_layer, 0, 1.0 / 16.0, 1, HQ)
    max_abs, max_rel = attention_error(load("attn"), ref)
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, (max_abs, max_rel)
