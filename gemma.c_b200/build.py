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

SOURCES = ["decode_attention.cu", "decode_balanced.cu", "decode_gqa16.cu", "decode_no_alloc.cu", "decode_projection.cu", "peer_gather.cu", "append_prep.cu", "prefill_attention.cu", "prefill_attention_sm100.cu", "fp8_cache.cu", "host_api.cu"]
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


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the CUDA sources into the shared library; returns its path."""
    if not force and is_current():
        return LIB_PATH
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    srcs = [str(CSRC / s) for s in SOURCES if (CSRC / s).exists()]
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd += [*srcs, "-o", str(tmp)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stderr)
    os.replace(tmp, LIB_PATH)
    STAMP_PATH.write_text(source_hash() + "\n")
    return LIB_PATH


if __name__ == "__main__":
    import sys

    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
