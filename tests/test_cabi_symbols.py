"""The C-ABI library loads without a GPU and exports every symbol ``include/emk.h`` declares (no compute calls)."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols() -> list[str]:
    text = (ROOT / "include" / "emk.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(emk_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_what_the_binding_binds(libemk):
    from deplodock_b200 import cabi

    declared = _declared_symbols()
    assert declared, "no declarations found in include/emk.h"
    assert sorted(cabi.EXPORTED_SYMBOLS) == declared


def test_library_exports_every_declared_symbol(libemk):
    lib = ctypes.CDLL(str(libemk))
    for name in _declared_symbols():
        assert hasattr(lib, name), f"libemk.so does not export {name}"


def test_version_and_status_strings(libemk):
    from deplodock_b200 import cabi

    lib = cabi.load_library()
    assert lib.emk_version() == 100
    assert lib.emk_status_string(cabi.EMK_OK) == b"ok"
    assert b"wait" in lib.emk_status_string(cabi.EMK_ERR_TIMEOUT)
    assert lib.emk_status_string(12345) == b"unknown status"


def test_no_torch_types_in_the_abi():
    text = (ROOT / "include" / "emk.h").read_text()
    assert 'extern "C"' in text
    code = re.sub(r"/\*.*?\*/", "", text, flags=re.S)  # declarations only: comments cite Torch-IR op names
    assert "torch" not in code.lower() and "at::" not in code and "Tensor" not in code


def test_null_handle_is_rejected_without_a_gpu(libemk):
    from deplodock_b200 import cabi

    lib = cabi.load_library()
    assert lib.emk_rmsnorm(None, None, None, None, 1, 1, 1e-6, 0, None) == cabi.EMK_ERR_ARG
    assert lib.emk_linear_bf16(None, None, None, None, None, 1, 8, 8, 0, 0, None) == cabi.EMK_ERR_ARG
    assert lib.emk_destroy(None) == cabi.EMK_ERR_ARG
