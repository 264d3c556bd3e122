"""ctypes binding of libb200attn.so (the C ABI declared in include/b200attn.h)."""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint64, c_void_p

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libb200attn.so")
_lib = None

# name -> (restype, argtypes); one entry per declaration in include/b200attn.h.
SIGNATURES = {
    "b200attn_version": (c_int, []),
    "b200attn_status_string": (c_char_p, [c_int]),
    "b200attn_paged_update_cache": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int,
         c_int, c_int, c_int, c_int, c_int64, c_void_p],
    ),
    "b200attn_paged_update_cache_ex": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int,
         c_int, c_int, c_int, c_int, c_int64, c_int, c_void_p],
    ),
    "b200attn_paged_fill_cache": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p,
         c_int, c_int, c_int, c_int, c_int, c_int64, c_void_p],
    ),
    "b200attn_paged_fill_cache_ex": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p,
         c_int, c_int, c_int, c_int, c_int, c_int64, c_int, c_void_p],
    ),
    "b200attn_kv_scatter_slots": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_int,
         c_int64, c_void_p],
    ),
    "b200attn_kv_scatter_slots_ex": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_int,
         c_int64, c_int, c_void_p],
    ),
    "b200attn_dequant_pages_fp8": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p,
         c_int, c_int, c_int, c_int, c_int64, c_void_p],
    ),
    "b200attn_build_step_metadata": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
         c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "b200attn_rope_kv_scatter_slots": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int,
         c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int64, c_void_p],
    ),
    "b200attn_paged_decode": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int,
         c_void_p, c_int, c_int, c_int, c_int, c_int, c_int64, c_float, c_int, c_int, c_void_p,
         c_size_t, c_void_p],
    ),
    "b200attn_paged_decode_ex": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int,
         c_void_p, c_int, c_int, c_int, c_int, c_int, c_int64, c_float, c_int, c_void_p, c_int,
         c_int, c_int, c_void_p, c_size_t, c_void_p],
    ),
    "b200attn_paged_decode_step": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
         c_int, c_void_p, c_int64, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int64,
         c_float, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p],
    ),
    "b200attn_paged_decode_static": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int,
         c_void_p, c_int, c_int, c_int, c_int, c_int, c_int64, c_float, c_int, c_int, c_void_p],
    ),
    "b200attn_decode_auto_splits": (c_int, [c_int, c_int, c_int, c_int]),
    "b200attn_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "b200attn_prefill": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int64, c_void_p,
         c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
         c_int64, c_float, c_void_p],
    ),
    "b200attn_prefill_ex": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int64, c_void_p,
         c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
         c_int64, c_float, c_int, c_void_p],
    ),
    "b200attn_comm_bytes": (c_size_t, [c_int, c_int, c_int]),
    "b200attn_rowlinear_plan": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p]),
    "b200attn_comm_alloc": (c_int, [c_size_t, c_void_p]),
    "b200attn_comm_free": (c_int, [c_void_p]),
    "b200attn_comm_export": (c_int, [c_void_p, c_void_p]),
    "b200attn_comm_import": (c_int, [c_void_p, c_void_p]),
    "b200attn_comm_close": (c_int, [c_void_p]),
    "b200attn_rowlinear_allreduce": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int,
         c_int, c_void_p, c_int, c_int, c_int, c_uint64, c_void_p],
    ),
    "b200attn_read_error_word": (c_int, [ctypes.POINTER(c_int32), c_void_p]),
    "b200attn_peek_error_word_async": (c_int, [c_void_p, c_void_p]),
}


class B200AttnError(RuntimeError):
    """A C-ABI entry point returned a non-zero status."""

    def __init__(self, fn: str, status: int):
        self.status = status
        text = lib().b200attn_status_string(status).decode()
        super().__init__(f"{fn} failed with status {status}: {text}")


def lib_path() -> str:
    return _LIB_PATH


def lib():
    """Loads the library once.  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(
                f"{_LIB_PATH} is missing; build it with `python -m b200attn.build` "
                "(b200attn has no CPU or PyTorch fallback)"
            )
        handle = ctypes.CDLL(_LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(fn: str, status: int) -> None:
    if status != 0:
        raise B200AttnError(fn, status)
