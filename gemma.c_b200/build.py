"""In-tree build of libgemma4_b200kv.so (sm_100a only) with nvcc.

The library is rebuilt when the hash of its sources changes; the built file
and its hash stamp live in ``_build/`` next to this module.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO_DIR = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR / "_build"
LIB_PATH = BUILD_DIR / "libgemma4_b200kv.so"
STAMP_PATH = BUILD_DIR / "libgemma4_b200kv.sha256"

SOURCES = ["decode_attention.cu", "decode_balanced.cu", "decode_pagetile.cu", "decode_gqa16.cu", "decode_no_alloc.cu", "decode_projection.cu", "peer_gather.cu", "bounded_wait.cu", "append_prep.cu", "prefill_attention.cu", "prefill_attention_sm100.cu", "fp8_cache.cu", "host_api.cu"]
NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "-shared",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the B200 KV library cannot be built")


def _source_files() -> list[Path]:
    files = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    files += sorted(CSRC.glob("*.cuh"))
    files += sorted((REPO_DIR / "include").glob("*.h*"))
    return files


def source_hash() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in _source_files():
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def is_current() -> bool:
    return (
        LIB_PATH.exists()
        and STAMP_PATH.exists()
        and STAMP_PATH.read_text().strip() == source_hash()
    )


def _object_key(src: Path) -> str:
    """Hash of what one object file depends on: its source, every header, the flags."""
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in [src, *sorted(CSRC.glob("*.cuh")), *sorted((REPO_DIR / "include").glob("*.h*"))]:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the CUDA sources into the shared library; returns its path. Every source becomes an
    object of its own (compiled in parallel, kept in ``_build/obj`` and reused while its hash holds),
    then one link."""
    if not force and is_current():
        return LIB_PATH
    from concurrent.futures import ThreadPoolExecutor

    obj_dir = BUILD_DIR / "obj"
    obj_dir.mkdir(parents=True, exist_ok=True)
    compile_flags = [f for f in NVCC_FLAGS if f != "-shared"]
    srcs = [CSRC / s for s in SOURCES if (CSRC / s).exists()]

    def compile_one(src: Path):
        obj, stamp = obj_dir / (src.stem + ".o"), obj_dir / (src.stem + ".sha256")
        key = _object_key(src)
        if not force and obj.exists() and stamp.exists() and stamp.read_text().strip() == key:
            return obj, ""
        cmd = [_nvcc(), *compile_flags, *(["-Xptxas", "-v"] if verbose else []), "-c", str(src), "-o", str(obj)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n" + proc.stdout + proc.stderr)
        stamp.write_text(key + "\n")
        return obj, proc.stderr

    with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
        results = list(pool.map(compile_one, srcs))
    if verbose:
        print("".join(log for _, log in results))
    tmp = LIB_PATH.with_suffix(".so.tmp")
    link = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
            *[str(o) for o, _ in results], "-o", str(tmp)]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc link failed:\n" + proc.stdout + proc.stderr)
    os.replace(tmp, LIB_PATH)
    STAMP_PATH.write_text(source_hash() + "\n")
    return LIB_PATH


if __name__ == "__main__":
    import sys

    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
