"""Test configuration: the ``gpu`` marker, import path, and a once-per-session build of ``libemk.so``.

``-m "not gpu"`` covers the oracle against the golden fixtures, the host-side logic and the C-ABI symbol table;
``-m gpu`` holds the parity tests proper, which call the kernels through the C ABI on a B200.
"""

from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def libemk():
    """Path of the built kernel library (built in-tree on first use when nvcc is available)."""
    from deplodock_b200 import build, cabi

    if not cabi.LIB_PATH.exists():
        build.build()
    return cabi.LIB_PATH


@pytest.fixture(scope="session")
def golden_dir() -> Path:
    return GOLDEN


def load_golden(name: str):
    import numpy as np

    data = np.load(GOLDEN / f"{name}.npz")
    ins = {k[4:]: data[k] for k in data.files if k.startswith("in__")}
    outs = {k[5:]: data[k] for k in data.files if k.startswith("out__")}
    return ins, outs
