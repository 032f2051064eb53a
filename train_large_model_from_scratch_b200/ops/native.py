"""ctypes binding of the sm_100a kernel library (`libtlm_b200.so`, built in-tree
by `build_ext.py` from `csrc/*.cu`).

The library exports plain C launchers that take device pointers, sizes and a
CUDA stream; this module wraps them into functions on torch tensors. Nothing
here falls back to another implementation: on a machine with a GPU a missing
or unloadable library is an error.
"""
from __future__ import annotations

import ctypes
import os

import torch

_LIB = None
_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "libtlm_b200.so")


class NativeError(RuntimeError):
    pass


def lib_path() -> str:
    return _LIB_PATH


def available() -> bool:
    return torch.cuda.is_available() and os.path.exists(_LIB_PATH)


def lib():
    global _LIB
    if _LIB is None:
        if not os.path.exists(_LIB_PATH):
            raise NativeError(
                f"{_LIB_PATH} not found: build it with `python -m train_large_model_from_scratch_b200.build_ext`")
        _LIB = ctypes.CDLL(_LIB_PATH)
        _declare(_LIB)
    return _LIB
