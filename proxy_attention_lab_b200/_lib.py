"""ctypes loader for libpal_b200.so, the C-ABI library that holds every CUDA kernel.

There is no fallback: if the library is missing or does not export a symbol the header
declares, importing this module raises.  Build it with ``python proxy_attention_lab_b200/build.py``.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libpal_b200.so"

PAL_OK = 0
PAL_ERR_BAD_ARG = -1
PAL_ERR_UNSUPPORTED = -2
PAL_ERR_LAUNCH = -3
PAL_ERR_WORKSPACE = -4
PAL_ERR_TIMEOUT = -5

PAL_DTYPE_F16 = 0
PAL_DTYPE_BF16 = 1
PAL_OUT_F32 = 0x100
PAL_STATIC_SCRATCH_BYTES = 16 * 1024 * 1024

PAL_DECODE_SINGLE_PASS = 0
PAL_DECODE_AUTO = -1

_P = c_void_p
# name -> (restype, argtypes); mirrors include/pal_b200.h one to one
SIGNATURES = {
    "pal_last_error": (c_char_p, []),
    "pal_version": (c_char_p, []),
    "pal_get_k_cache_stripe_size": (c_int, [c_int]),
    "pal_get_optimal_page_size": (c_int, []),
    "pal_get_k_cache_shape": (c_int, [c_int64, c_int, c_int, c_int, c_int, ctypes.POINTER(c_int64)]),
    "pal_get_v_cache_shape": (c_int, [c_int64, c_int, c_int, c_int, c_int, ctypes.POINTER(c_int64)]),
    "pal_fill_kv_pages": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int64, c_int, c_int, c_int, c_int, c_int64, c_int, c_int, _P]),
    "pal_fill_kv_pages_slots": (c_int, [_P, _P, _P, _P, _P, c_int64, c_int, c_int, c_int, c_int64, c_int, _P]),
    "pal_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    "pal_decode_auto_partition_pages": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int]),
    "pal_paged_attention_decode": (
        c_int,
        [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int64, c_int, c_float, c_int, c_int, _P, c_size_t, _P],
    ),
    "pal_paged_attention_decode_append": (
        c_int,
        [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int64, c_int, c_float, c_int, c_int, _P, c_size_t, _P],
    ),
    "pal_paged_attention_decode_static": (
        c_int,
        [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int64, c_int, c_float, c_int, c_int, _P],
    ),
    "pal_paged_attention_decode_partials": (
        c_int,
        [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int64, c_int, c_float, c_int, c_int, _P, c_size_t, _P],
    ),
    "pal_lse_combine": (c_int, [_P, _P, _P, _P, c_int, c_int64, c_int, c_int, _P]),
    "pal_prefill_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "pal_paged_attention_prefill": (
        c_int,
        [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int64, c_int, c_float, c_int, c_int, _P, c_size_t, _P],
    ),
    "pal_paged_attention_prefill_ragged": (
        c_int,
        [_P, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int64, c_int, c_int, c_int, c_int, c_int, c_int64, c_int, c_float, c_int, c_int, _P, c_size_t, _P],
    ),
    "pal_paged_attention_decode_partials_packed": (
        c_int,
        [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int64, c_int, c_float, c_int, c_int, _P, c_size_t, _P],
    ),
    "pal_exchange_bytes": (c_size_t, [c_int, c_int64, c_int]),
    "pal_paged_attention_decode_ctx_exchange": (
        c_int,
        [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int64, c_int, c_float, c_int, c_int, _P, c_size_t,
         ctypes.POINTER(c_void_p), c_int, c_int, c_int64, _P],
    ),
    "pal_lse_combine_packed": (c_int, [_P, _P, c_int, c_int64, c_int, c_int, _P]),
    "pal_workspace_init": (c_int, [_P, c_size_t, _P]),
    "pal_set_wait_limit_cycles": (c_int64, [c_int64]),
    "pal_selftest_bounded_wait": (c_int, [_P, c_int64, _P]),
    "pal_check_status": (c_int, [_P, _P]),
    "pal_static_scratch_init": (c_int, []),
    "pal_check_status_static": (c_int, [_P]),
}


def _load() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} not found: the CUDA library has not been built "
            "(run `python proxy_attention_lab_b200/build.py`); there is no CPU fallback"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:  # pragma: no cover - a stale library
            raise ImportError(f"{LIB_PATH} does not export {name}; rebuild it") from e
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


def last_error() -> str:
    msg = lib.pal_last_error()
    return msg.decode() if msg else ""


def check(rc: int) -> None:
    """Turn a C-ABI return code into the exception the reference binding would raise."""
    if rc == PAL_OK:
        return
    msg = last_error() or f"pal_b200 error {rc}"
    if rc == PAL_ERR_BAD_ARG:
        raise ValueError(msg)
    raise RuntimeError(msg)
