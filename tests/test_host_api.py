"""CPU-only checks of the product library: it loads, exports every symbol the header declares,
and its host-side logic (geometry, page bookkeeping, RoPE tables, split planning) agrees with
the oracle. No device call is made here."""
from __future__ import annotations

import re
import subprocess
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parent.parent
HEADER = REPO / "include" / "gemma4_b200kv.h"


def _declared_in_header() -> set[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    names = set(re.findall(r"\b((?:b200kv|gemma4)_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol(kv):
    lib = kv.load_library()
    declared = _declared_in_header()
    assert declared, "no declarations parsed from the header"
    assert declared == set(kv.declared_symbols())
    nm = subprocess.run(["nm", "-D", "--defined-only", str(kv.library_path())], capture_output=True, text=True)
    exported = {line.split()[-1] for line in nm.stdout.splitlines() if line.strip()}
    for name in declared:
        assert name in exported, name
        assert getattr(lib, name) is not None
    assert lib.b200kv_compiled_arch() == 1000


def test_make_config_and_layer_index_match_oracle(kv, orc):
    for is_global in (False, True):
        a = kv.make_config(is_global, 130, 16, 65)
        b = orc.make_config(is_global, 130, 16, 65)
        assert a.astuple() == tuple(getattr(b, n) for n, _ in b._fields_)
    # five sliding layers then one global, and the last layer is global (src/gemma4.h:105-108)
    pattern = [kv.is_global_layer(i) for i in range(48)]
    assert pattern == [((i + 1) % 6 == 0) or i == 47 for i in range(48)]
    assert sum(pattern) == 8
    for layer in range(-1, 49):
        for g in (False, True):
            assert kv.layer_index(layer, g) == orc.lib().orc_layer_index(layer, int(g))
    assert kv.layer_index(5, True) == 0 and kv.layer_index(11, True) == 1 and kv.layer_index(6, False) == 5
    assert kv.layer_index(5, False) == -1


def test_cache_offset_matches_oracle(kv, orc):
    rng = np.random.default_rng(0)
    for _ in range(200):
        cfg = kv.make_kv_config(*(int(x) for x in rng.integers(1, 40, size=8)))
        idx = [int(rng.integers(0, 30)) for _ in range(5)]
        assert kv.cache_offset(cfg, *idx) == orc.cache_offset(cfg, *idx)
    big = kv.make_kv_config(8, 70000, 16, 2049, 64, 8, 256, 0)
    assert kv.cache_offset(big, 7, 69999, 15, 7, 255) == 8 * 70000 * 16 * 8 * 256 - 1   # needs int64


def test_ensure_page_and_range_match_oracle(kv, orc):
    rng = np.random.default_rng(1)
    for trial in range(30):
        page_size = int(rng.choice([1, 2, 4, 16, 64]))
        mpps = int(rng.integers(1, 9))
        batch = int(rng.integers(1, 4))
        window = int(rng.choice([0, page_size * mpps]))
        cfg = kv.make_kv_config(1, batch * mpps, page_size, mpps, batch, 2, 16, window)
        ta = np.full(batch * mpps, -1, dtype=np.int32); sa = ta.copy()
        tb = ta.copy(); sb = ta.copy()
        for _ in range(60):
            b = int(rng.integers(0, batch))
            pos = int(rng.integers(0, page_size * mpps * 3))
            if rng.random() < 0.5:
                ra = kv.ensure_page(ta, sa, cfg, b, pos)
                rb = orc.ensure_page(tb, sb, cfg, b, pos)
            else:
                n = int(rng.integers(0, 2 * page_size + 2))
                ra = kv.ensure_range(ta, sa, cfg, b, pos, n)
                rb = orc.ensure_range(tb, sb, cfg, b, pos, n)
            assert ra == rb
            assert np.array_equal(ta, tb) and np.array_equal(sa, sb)


def test_stale_slot_is_refused(kv):
    """src/gemma4_kv_cache.cu:117: a slot that already holds a later logical page rejects an
    earlier one; the tables stay as they were."""
    cfg = kv.make_kv_config(1, 2, 4, 2, 1, 1, 16, 8)
    table = np.full(2, -1, dtype=np.int32); slots = table.copy()
    assert kv.ensure_page(table, slots, cfg, 0, 9) == 0      # logical page 2 -> slot 0
    before = (table.copy(), slots.copy())
    assert kv.ensure_page(table, slots, cfg, 0, 1) == -1     # logical page 0 -> slot 0, stale
    assert np.array_equal(table, before[0]) and np.array_equal(slots, before[1])
    assert kv.ensure_range(table, slots, cfg, 0, 0, 0) == 0  # empty range is fine
    assert kv.ensure_range(table, slots, cfg, 0, 0, 6) == -1


def test_sliding_pages_per_sequence(kv, orc):
    for max_seq in (1, 4, 66, 1024, 1025, 5000):
        for page in (1, 2, 16, 64):
            assert kv.sliding_pages_per_sequence(max_seq, page) == orc.lib().orc_sliding_pages_per_sequence(max_seq, page)
    assert kv.sliding_pages_per_sequence(66, 64) == 2
    assert kv.sliding_pages_per_sequence(4096, 16) == 65 and kv.sliding_pages_per_sequence(4096, 64) == 17


@pytest.mark.parametrize("half,theta,exp_dim", [(128, 10000.0, 256), (64, 1000000.0, 512), (128, 1000000.0, 256)])
def test_rope_tables_bit_exact_with_oracle(kv, orc, half, theta, exp_dim):
    a = kv.fill_rope_tables(300, half, theta, exp_dim)
    b = orc.fill_rope_tables(300, half, theta, exp_dim)
    assert np.array_equal(a[0].view(np.uint32), b[0].view(np.uint32))
    assert np.array_equal(a[1].view(np.uint32), b[1].view(np.uint32))


def test_plan_splits_and_workspace(kv):
    for batch, keys, heads in ((1, 1024, 8), (1, 4096, 8), (64, 32768, 8), (1, 131072, 8), (1, 131072, 1), (32, 8192, 8)):
        size, count = kv.plan_splits(batch, keys, heads, 148)
        tile = (16 // heads) * 4
        assert size % tile == 0 and size >= tile
        assert (count - 1) * size < keys <= count * size
    assert kv.plan_splits(1, 0, 8, 148)[1] == 1
    m, l, acc = kv.decode_workspace_bytes(64, 16, 256, 128)
    assert (m, l, acc) == (64 * 16 * 128 * 4,) * 2 + (64 * 16 * 128 * 256 * 4,)
    assert kv.decode_workspace_bytes(64, 16, 256, 1) == (0, 0, 0)


def test_host_argument_rejection_needs_no_device(kv):
    """Bad host arguments return cudaErrorInvalidValue before any launch
    (src/gemma4_kv_cache.cu:162-173); an empty write is a success (:161)."""
    cfg = kv.make_kv_config(1, 2, 4, 2, 1, 2, 16, 0)
    assert kv.kv_cache_write(None, None, cfg, None, None, None, 0, 0, None, None, stream=0, check=False) == 0
    assert kv.kv_cache_write(None, None, cfg, None, None, None, 1, 0, None, None, stream=0, check=False) == 1
    bad = kv.make_kv_config(1, 2, 4, 2, 1, 2, 12, 0)     # head_dim not a multiple of 8
    assert kv.kv_cache_write(16, 16, bad, 16, 16, 16, 1, 0, 16, 16, stream=0, check=False) == 1
    assert kv.kv_cache_write(16, 16, cfg, 16, 16, 16, 1, 1, 16, 16, stream=0, check=False) == 1   # layer out of range
    assert kv.kv_cache_write(16, 16, cfg, 16, 16, 16, -1, 0, 16, 16, stream=0, check=False) == 1
    good = kv.make_kv_config(1, 64, 16, 64, 1, 8, 256, 1024)
    args = dict(cache_layer=0, softmax_scale=1 / 16, split_size=64, num_splits=16, batch_count=1, q_heads=16,
                stream=0, check=False)
    assert kv.decode_attention(None, None, 16, 16, 16, good, 16, 16, **args) == 1          # null output
    assert kv.decode_attention(16, None, 16, 16, 16, good, 16, 16, **args) == 1            # splits without scratch
    tight = kv.make_kv_config(1, 32, 16, 32, 1, 8, 256, 1024)                               # ring < window
    assert kv.decode_attention(16, None, 16, 16, 16, tight, 16, 16, **{**args, "num_splits": 1}) == 1
    odd = kv.make_kv_config(1, 64, 16, 64, 1, 3, 256, 0)                                    # unknown geometry
    assert kv.decode_attention(16, None, 16, 16, 16, odd, 16, 16, **{**args, "num_splits": 1, "q_heads": 6}) == 1
    assert kv.decode_attention(16, None, 16, 16, 16, good, 16, 16, **{**args, "num_splits": 1, "softmax_scale": 0.0}) == 1
    assert kv.decode_append(None, 16, 16, good, 16, 16, 0, 16, 16, 16, 16, 16, 16, 16, 1, 16, 256, stream=0, check=False) == 1
    assert kv.decode_append(16, 16, 16, good, 16, 16, 0, 16, 16, 16, 16, 16, 16, 16, 1, 16, 100, stream=0, check=False) == 1
    assert kv.decode_append(16, 16, 16, good, 16, 16, 0, 16, 16, 16, 16, 16, 16, 16, 0, 16, 256, stream=0, check=False) == 0


def test_projection_and_peer_argument_rejection_needs_no_device(kv):
    """The decode projections and the peer-memory exchange reject bad host arguments before any CUDA call;
    zero rows is a success without a launch."""
    a = kv.IngressArgs()
    assert kv.decode_ingress(a, stream=0, check=False) == 0
    a.batch_count, a.hidden_size, a.cols, a.q_width, a.k_width = 1, 3840, 8192, 4096, 2048
    assert kv.decode_ingress(a, stream=0, check=False) == 1                      # null pointers
    a.raw_qkv = a.x = a.input_norm_weight = a.qkv_proj_col_major = 4096
    a.hidden_size = 4096
    assert kv.decode_ingress(a, stream=0, check=False) == 1                      # hidden size the kernel is not built for
    a.hidden_size, a.x = 3840, 4100
    assert kv.decode_ingress(a, stream=0, check=False) == 1                      # misaligned row
    a.x, a.q_width, a.k_width = 4096, 8192, 2048
    assert kv.decode_ingress(a, stream=0, check=False) == 1                      # q + k wider than the projection
    e = kv.EgressArgs()
    assert kv.decode_egress(e, stream=0, check=False) == 0
    e.batch_count, e.hidden_size, e.attention_width = 1, 3840, 4096
    assert kv.decode_egress(e, stream=0, check=False) == 1                       # null pointers
    for name, _ in kv.EgressArgs._fields_[:10]:
        setattr(e, name, 4096)
    e.attention_width = 1024
    assert kv.decode_egress(e, stream=0, check=False) == 1                       # width other than 4096 / 8192
    e.attention_width, e.ffn_x, e.pre_ffn_norm_weight = 4096, 4096, None
    assert kv.decode_egress(e, stream=0, check=False) == 1                       # ffn_x without its norm weight
    layer = kv.AttentionLayerArgs()
    layer.kv.batch_count = 1
    assert kv.decode_attention_layer(layer, stream=0, check=False) == 1          # no geometry, no scratch
    with pytest.raises(kv.CudaError):
        kv.PeerBuffer(1000, 2, 0)                                                # slot not a multiple of 16
    with pytest.raises(kv.CudaError):
        kv.PeerBuffer(1024, 2, 2)                                                # rank outside the world
    with pytest.raises(kv.CudaError):
        kv.PeerBuffer(1024, 9, 0)                                                # more than 8 ranks


def _compile_and_run_binding(kv, tmp_path, extra):
    import shutil

    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    repo = kv.library_path().parents[2]
    exe = tmp_path / "megakernel_binding"
    lib_dir = kv.library_path().parent
    build = subprocess.run([nvcc, "-std=c++17", *extra, "-I", str(repo / "include"),
                            str(repo / "tests" / "cpp" / "megakernel_binding.cu"),
                            "-L", str(lib_dir), "-lgemma4_b200kv", "-Xlinker", "-rpath", "-Xlinker", str(lib_dir),
                            "-o", str(exe)], capture_output=True, text=True)
    assert build.returncode == 0, build.stdout + build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0, run.stdout + run.stderr
    assert run.stdout.split() == ["1", "1", "0"]


def test_cpp_header_binds_a_reference_shaped_layer_struct(kv, tmp_path):
    """include/gemma4_b200kv.hpp from a C++ translation unit: a struct with the member names of the reference's
    Gemma4DecodeMegakernelLayerArgs goes through the header's binding template and links against the library."""
    _compile_and_run_binding(kv, tmp_path, [])


def _gemma_c_src():
    import os

    src = os.environ.get("GEMMA_REF_SRC") or str(Path(__file__).resolve().parents[2] / "reference" / "src")
    return src if Path(src, "gemma4_megakernel.cuh").is_file() else None


@pytest.mark.skipif(_gemma_c_src() is None, reason="gemma.c sources not mounted")
def test_cpp_header_sits_on_top_of_the_reference_headers(kv, tmp_path):
    """The same translation unit with the reference's real gemma4_megakernel.cuh (which pulls in its own
    gemma4_runtime.cuh and gemma4_kv_cache.cuh): the library's header adds its entry points on top without
    redefining a type, its layout static_asserts hold for the reference's structs, and the reference's
    Gemma4DecodeMegakernelLayerArgs binds."""
    _compile_and_run_binding(kv, tmp_path, ["-DB200KV_TEST_WITH_GEMMA_C", "-I", _gemma_c_src()])


@pytest.mark.skipif(_gemma_c_src() is None, reason="gemma.c sources not mounted")
def test_reference_tests_compile_against_the_stand_in_headers(kv, tmp_path):
    """The reference's own test programs, unchanged, compile against include/compat (ahead of the reference's src/
    on the include path) and link to the library alone -- every symbol they need is exported with the
    reference's signature. They run on a GPU in tests/test_gpu_reference_boundary.py."""
    import shutil

    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    repo = kv.library_path().parents[2]
    lib_dir = kv.library_path().parent
    tests = Path(_gemma_c_src()).parent / "tests"
    for name in ("test_kv_cache", "test_runtime_state"):
        build = subprocess.run([nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
                                "-I", str(repo / "include" / "compat"), "-I", str(repo / "include"),
                                "-I", _gemma_c_src(), str(tests / f"{name}.cu"), "-L", str(lib_dir),
                                "-lgemma4_b200kv", "-o", str(tmp_path / name)], capture_output=True, text=True)
        assert build.returncode == 0, name + "\n" + build.stdout + build.stderr


def test_partition_helpers_of_the_c_abi(kv):
    """b200kv_shard_sequences / b200kv_kv_head_range / b200kv_key_range_page_table called directly: every sequence
    owned once, rank loads within one sequence of each other, heads dealt in equal runs, a key range's page-table
    view starts at local position 0; arguments that make no sense return -1."""
    import ctypes

    lib = kv.load_library()
    rng = np.random.default_rng(4)
    keys = rng.integers(512, 32769, size=64).astype(np.int64)
    for world in (1, 2, 4, 8):
        owner = np.full(64, -1, np.int32)
        assert lib.b200kv_shard_sequences(keys.ctypes.data, 64, world, owner.ctypes.data) == 0
        assert owner.min() == 0 and owner.max() == world - 1
        loads = np.array([keys[owner == r].sum() for r in range(world)])
        assert loads.max() - loads.min() <= keys.max()
    assert lib.b200kv_shard_sequences(keys.ctypes.data, 64, 0, owner.ctypes.data) == -1
    first, count = ctypes.c_int32(), ctypes.c_int32()
    assert lib.b200kv_kv_head_range(8, 4, 3, ctypes.byref(first), ctypes.byref(count)) == 0
    assert (first.value, count.value) == (6, 2)
    assert lib.b200kv_kv_head_range(8, 3, 0, ctypes.byref(first), ctypes.byref(count)) == -1
    table = (np.arange(10, dtype=np.int32) + 100)
    out = np.zeros(10, np.int32)
    length, start = ctypes.c_int32(), ctypes.c_int32()
    assert lib.b200kv_key_range_page_table(table.ctypes.data, 10, 150, 16, 4, 3, out.ctypes.data,
                                           ctypes.byref(length), ctypes.byref(start)) == 0
    assert (length.value, start.value, out[0], out[1]) == (6, 144, 109, -1)
    assert lib.b200kv_key_range_page_table(table.ctypes.data, 10, 150, 16, 4, 4, out.ctypes.data,
                                           ctypes.byref(length), ctypes.byref(start)) == -1


def _step_entries(kv, specs):
    """LayerStepArgs array for the planning call; specs: (cache pointer, cache layer, batch, window) per entry.
    Nothing is dereferenced by b200kv_decode_step_plan, so the pointers are just distinct numbers."""
    arr = (kv.LayerStepArgs * len(specs))()
    for a, (cache, layer, batch, window) in zip(arr, specs):
        pages = 64 if window else 2048
        a.cache_config = kv.make_kv_config(4, max(batch, 1) * pages, 16, pages, max(batch, 1), 8, 256, window)
        a.cache_k, a.cache_v, a.cache_layer = cache, cache + 0x1000, layer
        a.batch_count, a.q_heads, a.rotary_dim, a.split_size, a.num_splits = batch, 16, 256, 0, 37
        a.ticket, a.raw_k, a.token_position = 0x7000, 0x5000, 0x6000
    return arr


def test_decode_step_plan_of_runs(kv):
    """The host logic behind b200kv_decode_step_bf16 (no device involved). Layers of a model in order: from the
    second entry on nothing in flight writes an entry's cache, entries release their successor at once, and a run
    is cut after six early releases. Steps of one layer: every entry allows for as many steps of its own layer in
    flight as the run is long. An entry that is not a one-launch layer-step ends the run on both sides."""
    n = 48
    held, early = kv.decode_step_plan(_step_entries(kv, [(0x100000, i % 4, 1, 1024) for i in range(n)]), n)
    assert held[0] == 1 and held[1:4] == [0, 0, 0]
    held, early = kv.decode_step_plan(_step_entries(kv, [(0x100000 * (i + 1), 0, 1, 1024) for i in range(n)]), n)
    assert held == [1] + [0] * (n - 1)
    assert early == [i % 7 != 0 and i + 1 < n for i in range(n)]

    n = 16                                               # sixteen steps of ONE layer (a one-layer decode loop)
    held, early, fwd = kv.decode_step_plan(_step_entries(kv, [(0x100000, 0, 1, 0)] * n), n, forwarded=True)
    assert early == [i % 7 != 0 and i + 1 < n for i in range(n)]
    assert held == [1, 1, 2, 3, 4, 5, 6, 7, 1, 2, 3, 4, 5, 6, 7, 1]
    # the first entry's predecessor is not an entry of the call: its rows cannot be prepared here
    assert fwd == [0] + held[1:]

    n = 8                                                # two layers in turn
    held, early, fwd = kv.decode_step_plan(_step_entries(kv, [(0x100000, i % 2, 2, 1024) for i in range(n)]), n,
                                           forwarded=True)
    assert held == [1, 0, 1, 1, 2, 2, 3, 3]
    assert fwd == [0, 0, 1, 1, 2, 2, 3, 3]
    assert early == [False, True, True, True, True, True, True, False]

    specs = [(0x100000 * (i + 1), 0, 1, 1024) for i in range(6)]
    specs[3] = (0x900000, 0, 64, 1024)                   # 64 sequences: the balanced kernel's job
    held, early = kv.decode_step_plan(_step_entries(kv, specs), 6)
    assert early == [False, True, False, False, True, False]
    assert held == [1, 0, 0, 0, 0, 0]
    arr = _step_entries(kv, [(0x100000 * (i + 1), 0, 1, 1024) for i in range(4)])
    for a in arr:
        a.ticket = None                                  # without tickets nothing runs as one launch
    held, early = kv.decode_step_plan(arr, 4)
    assert early == [False] * 4 and held == [1, 0, 0, 0]
    assert kv.decode_step_plan(arr, 0) == ([], [])


def test_device_phase_header_compiles_into_a_kernel_of_its_own(tmp_path):
    """include/gemma4_b200kv_device.cuh is header-only: the cooperative harness kernel that calls its three
    phases builds with nvcc for sm_100a without the library (no GPU needed here; the GPU test runs it)."""
    from tests.gpu_util import build_device_phases_harness

    lib = build_device_phases_harness(force=True)
    assert lib.exists() and lib.stat().st_size > 0
    exported = subprocess.run(["nm", "-D", "--defined-only", str(lib)], capture_output=True, text=True).stdout
    assert "device_phases_layer_step" in exported


@pytest.mark.skipif(_gemma_c_src() is None, reason="gemma.c sources not mounted")
def test_device_phase_header_inside_a_gemma_c_translation_unit(tmp_path):
    """include/gemma4_b200kv_device.cuh in a translation unit that has the reference's own headers (the situation
    of its decode megakernel): with GEMMA4_B200KV_USE_REFERENCE_HEADERS the library's header declares no type
    of its own, and a kernel that calls the three phases with the reference's Gemma4KvCacheConfig compiles."""
    import shutil

    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    repo = Path(__file__).resolve().parents[1]
    src = tmp_path / "phases_in_gemma_c.cu"
    src.write_text('''
#include "gemma4_kv_cache.cuh"   // gemma.c's own
#include "gemma4_b200kv_device.cuh"
__global__ void layer(__nv_bfloat16 *q_prepared, __nv_bfloat16 *cache_k, __nv_bfloat16 *cache_v,
                      __nv_bfloat16 *out, float *pm, float *pl, float *pacc, Gemma4KvCacheConfig cfg,
                      const int32_t *table, const int32_t *pos, const int32_t *len, const __nv_bfloat16 *q,
                      const __nv_bfloat16 *k, const __nv_bfloat16 *v, const __nv_bfloat16 *w, const float *cs) {
  extern __shared__ float smem[];
  b200kv_device::append_phase(q_prepared, cache_k, cache_v, cfg, table, pos, 0, q, k, v, w, w, cs, cs, 16,
                              int(blockIdx.x), int(blockIdx.y), int(threadIdx.x), int(blockDim.x));
  b200kv_device::split_phase(pm, pl, pacc, out, nullptr, q_prepared, cache_k, cache_v, cfg, table, len, 0,
                             0.0625f, 20, 4, 16, int(blockIdx.x), int(blockIdx.y), int(blockIdx.z), smem,
                             int(threadIdx.x), int(blockDim.x));
  b200kv_device::reduce_phase(out, nullptr, pm, pl, pacc, cfg, len, 20, 4, 16, int(blockIdx.x),
                              int(blockIdx.y), int(threadIdx.x), int(blockDim.x));
}
''')
    build = subprocess.run([nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-c",
                            "-DGEMMA4_B200KV_USE_REFERENCE_HEADERS", "-I", _gemma_c_src(), "-I",
                            str(repo / "include"), str(src), "-o", str(tmp_path / "phases.o")],
                           capture_output=True, text=True)
    assert build.returncode == 0, build.stdout + build.stderr
