"""ctypes binding of libb200ta.so, the C ABI declared in ``include/b200ta.h``.

The library is the only compute backend: if it is missing, or a call returns a
non-zero status, this module raises — there is no PyTorch or CPU fallback.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p, POINTER
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = Path(os.environ.get("B200TA_LIBRARY", _PKG / "libb200ta.so"))

OK = 0
ERR_INVALID = -1
ERR_CUDA = -2
ERR_DRIVER = -3
ERR_DEVICE_WAIT = -4
ERR_UNSUPPORTED = -5

DTYPE_BF16 = 0
DTYPE_F32 = 1
EMPTY_ROW_ZEROS = 0
EMPTY_ROW_UNIFORM = 1

# name -> (restype, argtypes); kept in the order of include/b200ta.h
SIGNATURES: dict[str, tuple] = {
    "b200ta_version": (c_int, []),
    "b200ta_last_error": (c_char_p, []),
    "b200ta_device_status": (c_int, [POINTER(c_int)]),
    "b200ta_reset_device_status": (c_int, []),
    "b200ta_node_pack_bytes": (c_size_t, []),
    "b200ta_transition_pack_bytes": (c_size_t, []),
    "b200ta_pack_node_weights": (c_int, [c_void_p] * 7 + [c_int, c_void_p, c_void_p]),
    "b200ta_pack_transition_weights": (c_int, [c_void_p] * 4 + [c_int, c_void_p, c_void_p]),
    "b200ta_pack_relu_transition_weights": (c_int, [c_void_p] * 6 + [c_int, c_void_p, c_void_p]),
    "b200ta_prologue": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_float, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int,
         c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p],
    ),
    "b200ta_attention": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
         c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_float, c_int, c_int, c_int,
         c_int, c_int, c_void_p],
    ),
    "b200ta_attention_masked": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
         c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p,
         c_float, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ),
    "b200ta_epilogue": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64,
         c_int64, c_int64, c_int, c_int, c_int, c_void_p],
    ),
    "b200ta_node_workspace_bytes": (c_size_t, [c_int, c_int]),
    "b200ta_node_forward": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_float, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p,
         c_int64, c_int64, c_int64, c_void_p, c_size_t, c_int, c_int, c_void_p],
    ),
    "b200ta_node_static_max_positions": (c_int, []),
    "b200ta_node_forward_static": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_float, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p,
         c_int64, c_int64, c_int64, c_int, c_int, c_void_p],
    ),
    "b200ta_transition": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_void_p, c_float, c_void_p, c_int64, c_int64, c_int, c_void_p],
    ),
    "b200ta_transition_relu": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_void_p, c_float, c_void_p, c_int64, c_int64, c_int, c_void_p],
    ),
    "b200ta_pack_pair_bias_weights": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_void_p, c_void_p]),
    "b200ta_pair_bias": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_float, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int,
         c_int, c_int, c_int, c_int, c_void_p],
    ),
    "b200ta_row_stats": (c_int, [c_void_p, c_int64, c_int64, c_int, c_float, c_void_p, c_void_p]),
    "b200ta_linear": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64,
         c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ),
    "b200ta_transition_scatter": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ),
    "b200ta_epilogue_scatter": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int, c_int,
         c_int, c_int, c_int, c_void_p],
    ),
    "b200ta_trimul_pack_bytes": (c_size_t, []),
    "b200ta_pack_trimul_weights": (c_int, [c_void_p] * 12 + [c_int, c_void_p, c_void_p]),
    "b200ta_trimul_project": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_float, c_void_p,
         c_int64, c_int, c_int, c_int, c_void_p],
    ),
    "b200ta_trimul_contract": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int64, c_void_p]),
    "b200ta_trimul_output": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_float,
         c_int, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_void_p],
    ),
}


class B200TAError(RuntimeError):
    """A libb200ta call returned a non-zero status."""

    def __init__(self, fn: str, code: int, message: str):
        super().__init__(f"{fn} failed with status {code}: {message}")
        self.code = code


_lib: ctypes.CDLL | None = None


def load() -> ctypes.CDLL:
    """Load libb200ta.so (once) and declare every exported function."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m bionemo_inference_runtime_b200.csrc.build` "
            "(needs nvcc); this package has no fallback path."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue  # reported by call(); test_abi checks the full export list
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    msg = load().b200ta_last_error()
    return msg.decode() if msg else ""


def call(name: str, *args) -> None:
    """Call a status-returning entry point and raise on failure."""
    fn = getattr(load(), name, None)
    if fn is None:
        raise B200TAError(name, ERR_UNSUPPORTED, "symbol not exported by libb200ta.so")
    code = fn(*args)
    if code != OK:
        exc = ValueError if code == ERR_INVALID else B200TAError
        if exc is ValueError:
            raise ValueError(f"{name}: {last_error()}")
        raise B200TAError(name, code, last_error())


def device_status() -> int:
    status = c_int(0)
    call("b200ta_device_status", ctypes.byref(status))
    return status.value


def reset_device_status() -> None:
    call("b200ta_reset_device_status")
