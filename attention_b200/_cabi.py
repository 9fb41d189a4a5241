"""ctypes binding of the C-ABI library declared in include/gqa_decode_b200.h and
include/mla_decode_b200.h."""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_size_t, c_void_p

from ._paths import LIB_PATH

_P = c_void_p

# name -> (restype, argtypes); mirrors the two headers one to one
SIGNATURES = {
    "gqa_b200_abi_version": (c_int, []),
    "gqa_b200_strerror": (ctypes.c_char_p, [c_int]),
    "gqa_b200_chunk_tokens": (c_int, [c_int, c_int]),
    "gqa_b200_max_chunks_per_seq": (c_int, [c_int, c_int, c_int]),
    "gqa_b200_auto_chunk_tokens": (c_int, [c_int, c_int, c_int, c_int, c_int]),
    "gqa_b200_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    "gqa_b200_workspace_control_bytes": (c_size_t, []),
    "gqa_b200_workspace_init": (c_int, [_P, c_size_t, _P]),
    "gqa_b200_decode": (c_int, [_P] * 6 + [c_int] * 5 + [c_int64, c_int, c_int, c_float, _P,
                                                          c_size_t, _P]),
    "gqa_b200_decode_ex": (c_int, [_P] * 6 + [c_int] * 5 + [c_int64, c_int, c_int, c_float, _P,
                                                             c_size_t, _P, c_int, c_int, c_int, c_int]),
    "gqa_b200_decode_static": (c_int, [_P] * 6 + [c_int] * 5 + [c_int64, c_int, c_int, c_float, _P]),
    "gqa_b200_decode_split": (c_int, [_P] * 6 + [c_int] * 5 + [c_int64, c_int, c_int, c_float,
                                                                c_int, _P, _P]),
    "gqa_b200_prefill": (c_int, [_P] * 6 + [c_int] * 7 + [c_float, c_int, c_int, _P]),
    "gqa_b200_prefill_tc_status": (c_int, [c_int]),
    "gqa_b200_kv_append": (c_int, [_P] * 6 + [c_int] * 4 + [c_int64, c_int, c_int, _P]),
    # include/mla_decode_b200.h
    "mla_b200_project": (c_int, [_P] * 3 + [c_int, c_int64] + [c_int] * 4 + [_P]),
    "mla_b200_latent_kv_write": (c_int, [_P] * 4 + [c_int64, c_int, c_int, c_int, _P]),
    "mla_b200_attend_workspace_bytes": (c_size_t, [c_int] * 8),
    "mla_b200_attend_ex_workspace_bytes": (c_size_t, [c_int] * 9),
    "mla_b200_attend": (c_int, [_P] * 8 + [c_int] * 6 + [c_int64, c_int, c_int, c_int, c_float, c_int,
                                                         _P, c_size_t, _P]),
    "mla_b200_attend_ex": (c_int, [_P] * 8 + [c_int] * 6 + [c_int64, c_int, c_int, c_int, c_float, c_int,
                                                            _P, c_size_t, _P, c_int, c_int]),
    "mla_b200_decode_workspace_bytes": (c_size_t, [c_int] * 8),
    "mla_b200_decode": (c_int, [_P] * 10 + [c_int] * 8 + [c_int64, c_int, c_int, c_int, c_float, c_int,
                                                          _P, c_size_t, _P]),
    "mla_b200_tc_status": (c_int, [c_int]),
}

_lib = None
_load_error: Exception | None = None


def load():
    """The loaded library, or raises the (cached) load failure."""
    global _lib, _load_error
    if _lib is not None:
        return _lib
    if _load_error is not None:
        raise _load_error
    try:
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
        return lib
    except (OSError, AttributeError) as exc:
        _load_error = ImportError(f"cannot load {LIB_PATH}: {exc}")
        raise _load_error


def load_error():
    """None if the library loads, else the exception."""
    try:
        load()
        return None
    except ImportError as exc:
        return exc


def strerror(code: int) -> str:
    return load().gqa_b200_strerror(int(code)).decode()
