"""Loader for libtacvq.so (the C ABI declared in include/tacvq.h).

The library is the only implementation: if it is missing, stale or the device
is not a B200-class GPU the calls raise - there is no CPU or PyTorch fallback.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_double, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

ABI_VERSION = 1
LIB_PATH = Path(__file__).resolve().parent / "libtacvq.so"

_lib = None

_SIGNATURES = {
    "tacvq_version": (c_int, []),
    "tacvq_status_string": (c_char_p, [c_int]),
    "tacvq_table_sqnorm": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "tacvq_encode_tensor_memory_timeouts": (c_int, [c_void_p]),
    "tacvq_encode": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int]
                     + [c_int] * 7 + [c_int64, c_int64, c_void_p]),
    "tacvq_encode_whitened": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_int] + [c_int] * 7 + [c_int64, c_int64, c_void_p]),
    "tacvq_decode": (c_int, [c_void_p, c_void_p, c_void_p, c_int] + [c_int] * 8 + [c_int64, c_int64, c_void_p]),
    "tacvq_codeword_grad": (c_int, [c_void_p, c_void_p, c_void_p] + [c_int] * 8 + [c_int64, c_int64, c_void_p]),
    "tacvq_attn_workspace_bytes": (c_size_t, [c_int] * 6),
    "tacvq_attn_decode": (c_int, [c_void_p] * 8 + [c_size_t, c_void_p, c_void_p] + [c_int] * 7 + [c_int64, c_void_p]),
    "tacvq_decode_step": (c_int, [c_void_p, c_void_p, c_void_p, c_int] + [c_void_p] * 6 + [c_int64, c_int64, c_void_p, c_size_t,
                                  c_void_p, c_void_p] + [c_int] * 8 + [c_int64, c_void_p]),
    "tacvq_decode_step_host": (c_int, [c_void_p, c_void_p, c_int] + [c_void_p] * 6 + [c_int64, c_int64, c_void_p, c_size_t,
                                       c_void_p, c_void_p] + [c_int] * 8 + [c_int64, c_int, c_void_p]),
    "tacvq_set_ranges": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "tacvq_attn_static_scratch_bytes": (c_size_t, []),
    "tacvq_attn_decode_static": (c_int, [c_void_p] * 7 + [c_void_p, c_void_p] + [c_int] * 7 + [c_int64, c_void_p]),
    "tacvq_attn_combine": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "tacvq_rope_table": (c_int, [c_void_p, c_int64, c_int, c_double, c_int64, c_void_p]),
    "tacvq_attn_decode_rotary": (c_int, [c_void_p] * 9 + [c_size_t, c_void_p, c_void_p] + [c_int] * 7 + [c_int64, c_void_p]),
}

EXPORTS = tuple(_SIGNATURES)


class TacvqError(RuntimeError):
    """A libtacvq call returned a non-zero status."""

    def __init__(self, call: str, status: int, text: str):
        super().__init__(f"{call} failed: status {status} ({text})")
        self.call, self.status = call, status


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it is absent or has another ABI version."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m tac_vq_kv_cache_b200.build` "
            "(needs nvcc; there is no fallback implementation)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means a stale library
        fn.restype = restype
        fn.argtypes = argtypes
    if lib.tacvq_version() != ABI_VERSION:
        raise RuntimeError(f"libtacvq.so has ABI version {lib.tacvq_version()}, expected {ABI_VERSION}; rebuild it")
    _lib = lib
    return lib


def check(call: str, status: int) -> None:
    if status != 0:
        raise TacvqError(call, status, load().tacvq_status_string(status).decode())
