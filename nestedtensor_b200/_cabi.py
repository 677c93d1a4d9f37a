"""ctypes binding of lib/libntb200.so — the same C ABI a non-Python host would bind.

The operator layer (csrc/dispatch.cpp) links the library directly; this module exists for
callers that hold raw device pointers (tests, the benchmark's C-ABI timing loop, foreign
runtimes).  There is no fallback: if the library is missing, ``load()`` raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_uint64, c_void_p

from . import _build

_LIB = None

# name -> (restype, argtypes); mirrors include/ntb200.h declaration by declaration
SIGNATURES = {
    "ntb200_status_string": (c_char_p, [c_int]),
    "ntb200_version": (c_int, []),
    "ntb200_pad_nd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int64, c_int64, c_void_p,
                              c_int, c_uint64, c_void_p]),
    "ntb200_unpad_nd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int64, c_int64, c_void_p,
                                c_int64, c_int, c_void_p]),
    "ntb200_mask_from_sizes": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int64, c_void_p, c_void_p]),
    "ntb200_pad_with_mask": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int64,
                                     c_int64, c_void_p, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "ntb200_sizes_from_padded": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p, c_int, c_int,
                                         c_uint64, c_void_p]),
    "ntb200_sizes_from_mask": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p]),
    "ntb200_offsets_workspace_bytes": (c_size_t, [c_int64]),
    "ntb200_offsets_from_sizes": (c_int, [c_void_p, c_int64, c_int, c_int64, c_int64, c_void_p, c_void_p,
                                          c_size_t, c_void_p]),
    "ntb200_offsets_static_max_batch": (c_int64, []),
    "ntb200_offsets_from_sizes_static": (c_int, [c_void_p, c_int64, c_int, c_int64, c_int64, c_void_p, c_void_p]),
    "ntb200_token_index": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "ntb200_gemm_bias": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int,
                                 c_void_p]),
    "ntb200_gemm_bias_act": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
                                     c_int, c_int, c_void_p]),
    "ntb200_layer_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "ntb200_add_bias_residual_layer_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p,
                                                    c_int64, c_int64, c_int, c_void_p]),
    "ntb200_add_bias_gelu": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "ntb200_pack_pointers": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p]),
    "ntb200_embedding": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "ntb200_transpose_ragged": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int64, c_int, c_void_p]),
    "ntb200_device_error_flags": (c_int, []),
    "ntb200_varlen_attention_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int, c_int, c_int]),
    "ntb200_varlen_attention": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int64,
                                        c_float, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "ntb200_varlen_cross_attention": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p,
                                              c_void_p, c_int64, c_int64, c_int, c_int, c_int64, c_float, c_int, c_int, c_void_p]),
    "ntb200_varlen_cross_attention_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int, c_int, c_int]),
    "ntb200_varlen_cross_attention_ws": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p,
                                                 c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_int64, c_float, c_int, c_int,
                                                 c_void_p, c_size_t, c_void_p]),
    "ntb200_varlen_attention_weights": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                                c_int64, c_int, c_int, c_int64, c_float, c_int, c_int, c_void_p]),
    "ntb200_add_qkv_bias_pad": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                        c_int, c_int, c_int64, c_int, c_void_p]),
    "ntb200_transpose_rm_padding": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int64,
                                            c_int, c_void_p]),
    "ntb200_softmax_masked": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_int64, c_int64, c_float, c_int,
                                      c_void_p]),
}

DTYPE_CODES = {"float32": 0, "float16": 1, "bfloat16": 2}


def lib_path() -> str:
    return _build.CABI_LIB


def load() -> ctypes.CDLL:
    """Load the kernel library and attach prototypes.  Raises if it has not been built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not os.path.exists(path):
        raise RuntimeError(
            "nestedtensor_b200: %s is missing — build it with `python -m nestedtensor_b200._build` "
            "(there is no CPU or eager fallback)" % path)
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib


class Ntb200Error(RuntimeError):
    def __init__(self, fn: str, status: int):
        self.status = status
        msg = load().ntb200_status_string(status).decode()
        super().__init__("%s failed: %s (%d)" % (fn, msg, status))


def check(fn: str, status: int) -> None:
    if status != 0:
        raise Ntb200Error(fn, status)


def host_i64(values):
    """A ctypes int64 array for the `h_*` (host pointer) parameters."""
    arr = (c_int64 * max(len(values), 1))(*[int(v) for v in values])
    return arr
