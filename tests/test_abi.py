"""The C-ABI library loads without a GPU and exports exactly what include/b200ta.h declares."""

import ctypes
import re
from pathlib import Path

import pytest

from bionemo_inference_runtime_b200 import _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "b200ta.h"


def declared_functions() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200ta_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for required in ("b200ta_prologue", "b200ta_attention", "b200ta_epilogue", "b200ta_transition",
                     "b200ta_pack_node_weights", "b200ta_pack_transition_weights", "b200ta_last_error"):
        assert required in names


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in b200ta.h but not exported: {missing}"


def test_python_signatures_cover_the_header():
    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_version_and_sizes_without_a_gpu():
    lib = _lib.load()
    assert lib.b200ta_version() >= 100
    assert lib.b200ta_node_pack_bytes() % 256 == 0 and lib.b200ta_node_pack_bytes() > 528 * 128 * 2
    assert lib.b200ta_transition_pack_bytes() % 256 == 0


def test_argument_validation_happens_before_any_cuda_call():
    """Bad arguments are refused with B200TA_ERR_INVALID and a message; nothing is launched."""
    lib = _lib.load()
    rc = lib.b200ta_transition(None, 128, None, None, 1e-5, None, 128, 16, 0, None)
    assert rc == _lib.ERR_INVALID
    assert "NULL" in _lib.last_error()
    with pytest.raises(ValueError):
        _lib.call("b200ta_epilogue", None, 0, 0, 0, None, None, 0, 0, 0, None, 0, 0, 0, 1, 1, 1, None)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(ImportError):
        _lib.load()
