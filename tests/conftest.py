"""Shared pytest fixtures: package loader, oracle handle, marker registration.

``gpu`` marks tests that need a B200; everything else runs on CPU only.
The package directory is named ``gemma.c_b200`` (a dot is not importable as a
plain module name), so it is loaded by path under the name ``gemma_c_b200``.
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))


def load_package():
    name = "gemma_c_b200"
    if name in sys.modules:
        return sys.modules[name]
    pkg_dir = REPO / "gemma.c_b200"
    spec = importlib.util.spec_from_file_location(
        name, pkg_dir / "__init__.py", submodule_search_locations=[str(pkg_dir)])
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def kv():
    """The product binding (C-ABI library loaded through ctypes)."""
    return load_package()


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle binding (test infrastructure)."""
    from oracle import binding

    binding.build()
    return binding
