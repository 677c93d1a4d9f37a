"""Loads the operator layer (lib/ntb200_dispatch.so) and exposes ``torch.ops.nestedtensor``.

There is no eager or CPU fallback: if the native libraries are missing the first operator
call raises with the build command.
"""
from __future__ import annotations

import os

import torch

from . import _build

_LOADED = False


def load() -> None:
    global _LOADED
    if _LOADED:
        return
    for path in (_build.CABI_LIB, _build.DISPATCH_LIB):
        if not os.path.exists(path):
            raise RuntimeError(
                "nestedtensor_b200: native library %s is missing — run `python -m nestedtensor_b200._build` "
                "(this package has no CPU or eager fallback)" % path)
    torch.ops.load_library(_build.DISPATCH_LIB)
    _LOADED = True


def ops():
    """The ``torch.ops.nestedtensor`` namespace, loading the library on first use."""
    load()
    return torch.ops.nestedtensor
