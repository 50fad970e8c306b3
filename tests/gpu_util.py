"""Helpers for the GPU tests: numpy <-> device transfers that never touch the values."""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

need_gpu = pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a CUDA device")

_SIGNED = {np.dtype(np.uint16): np.int16, np.dtype(np.uint32): np.int32}


def dev(a: np.ndarray) -> torch.Tensor:
    """Copy a numpy array to the device bit for bit (uint16 travels as int16)."""
    a = np.ascontiguousarray(a)
    if a.dtype in _SIGNED:
        a = a.view(_SIGNED[a.dtype])
    return torch.from_numpy(a).cuda()


def host_u16(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16).reshape(-1)


def host_u8(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.uint8).numpy().reshape(-1)


def read_device(ptr: int, count: int, dtype) -> np.ndarray:
    """Read `count` elements from a raw device pointer owned by the library."""
    dt = {np.int32: torch.int32, np.float32: torch.float32}[dtype]
    out = torch.empty(count, dtype=dt, device="cuda")
    torch.cuda.synchronize()
    libcudart = ctypes.CDLL("libcudart.so.12")
    libcudart.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    rc = libcudart.cudaMemcpy(out.data_ptr(), ptr, count * out.element_size(), 3)  # device to device
    assert rc == 0, f"cudaMemcpy failed: {rc}"
    return out.cpu().numpy()


# --------------------------------------------------------------------------- harness of the device-side phases
HARNESS_SRC = Path(__file__).resolve().parent / "cpp" / "device_phases_harness.cu"
HARNESS_LIB = Path(__file__).resolve().parent / "_build" / "libdevice_phases_harness.so"


def build_device_phases_harness(force: bool = False) -> Path:
    """Compiles tests/cpp/device_phases_harness.cu (a cooperative kernel that calls nothing but the __device__
    phases of include/gemma4_b200kv_device.cuh) for sm_100a into tests/_build/. nvcc only, no GPU needed."""
    header = HARNESS_SRC.parents[2] / "include" / "gemma4_b200kv_device.cuh"
    newest = max(HARNESS_SRC.stat().st_mtime, header.stat().st_mtime)
    if not force and HARNESS_LIB.exists() and HARNESS_LIB.stat().st_mtime >= newest:
        return HARNESS_LIB
    HARNESS_LIB.parent.mkdir(exist_ok=True)
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
           "-Xcompiler", "-fPIC", str(HARNESS_SRC), "-o", str(HARNESS_LIB)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("device-phase harness did not build:\n" + proc.stderr[-3000:])
    return HARNESS_LIB
