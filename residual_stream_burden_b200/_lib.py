"""ctypes binding of the C ABI declared in ``include/sihc_b200.h``.

The shared library is built in-tree (``csrc/libsihc_b200.so``, see
``csrc/Makefile``).  There is deliberately no fallback: if the library is
missing or an entry point cannot be resolved, importing this module raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_uint64, c_void_p, POINTER

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libsihc_b200.so")

F32, BF16 = 0, 1
MAX_EVENTS = 24

# name -> (restype, argtypes); mirrors include/sihc_b200.h one to one
_GEOM = [c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]   # batch, grid, kh, kw, channels, dtype, wdtype, stream
SIGNATURES = {
    "sihc_version": (c_int, []),
    "sihc_status_string": (c_char_p, [c_int]),
    "sihc_read_fwd": (c_int, [c_void_p, c_void_p, POINTER(c_void_p), c_int] + _GEOM),
    "sihc_write_fwd": (c_int, [c_void_p, POINTER(c_void_p), c_void_p, c_void_p, c_int] + _GEOM),
    "sihc_write_read_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p] + _GEOM),
    "sihc_write_read_bwd_workspace_bytes": (c_size_t, [c_int64, c_int, c_int, c_int, c_int, c_int]),
    "sihc_write_read_bwd": (c_int, [c_void_p] * 9 + [c_void_p, c_size_t] + _GEOM),
    "sihc_wgrad_workspace_bytes": (c_size_t, [c_int, c_int64, c_int, c_int, c_int, c_int, c_int]),
    "sihc_read_bwd": (c_int, [c_void_p, POINTER(c_void_p), c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int] + _GEOM),
    "sihc_read_bwd_static": (c_int, [c_void_p, POINTER(c_void_p), c_void_p, c_void_p, c_void_p, c_int] + _GEOM),
    "sihc_write_bwd": (c_int, [c_void_p, POINTER(c_void_p), c_void_p, POINTER(c_void_p), c_void_p, c_void_p, c_size_t, c_int] + _GEOM),
    "sihc_tri_fwd": (c_int, [c_void_p, POINTER(c_void_p), c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_void_p]),
    "sihc_tri_workspace_bytes": (c_size_t, [c_int, c_int64, c_int, c_int]),
    "sihc_tri_bwd": (c_int, [c_void_p, POINTER(c_void_p), c_void_p, POINTER(c_void_p), c_void_p, c_void_p, c_size_t,
                             c_int, c_int64, c_int, c_int, c_int, c_void_p]),
    "sihc_tri_dgamma_workspace_bytes": (c_size_t, [c_int, c_int64, c_int, c_int]),
    "sihc_tri_dgamma": (c_int, [POINTER(c_void_p), POINTER(c_void_p), c_void_p, c_void_p, c_size_t, c_int, c_int64, c_int,
                                c_int, c_void_p]),
    "sihc_tune": (c_int, [c_char_p, c_int]),
    "sihc_probe_store_stream": (c_int, [c_void_p, c_size_t, c_void_p]),
    "sihc_launch_count": (c_uint64, []),
}


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C {os.path.join(_HERE, 'csrc')}` "
            "(nvcc, sm_100a). This package has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


class SihcError(RuntimeError):
    """A C ABI call returned a non-zero status."""


def check(status: int, what: str) -> None:
    if status != 0:
        text = lib.sihc_status_string(status)
        raise SihcError(f"{what} failed with status {status}: {text.decode() if text else '?'}")


def ptr_array(ptrs):
    """Host array of device pointers (None -> NULL)."""
    return (c_void_p * len(ptrs))(*ptrs)


def tune(name: str, value: int) -> None:
    check(lib.sihc_tune(name.encode(), int(value)), f"sihc_tune({name})")


def launch_count() -> int:
    return int(lib.sihc_launch_count())
