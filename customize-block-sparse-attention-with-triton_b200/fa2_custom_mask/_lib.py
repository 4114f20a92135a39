"""ctypes binding of libbsattn.so, the C-ABI CUDA library (see include/bsattn.h).

There is no fallback: if the shared library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbsattn.so")

BSA_F16, BSA_BF16 = 0, 1

_lib = None


class BsaError(RuntimeError):
    """A libbsattn entry point returned a negative status."""

    def __init__(self, fn: str, status: int, text: str):
        super().__init__(f"{fn} failed with status {status}: {text}")
        self.status = status


class ListSizes(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in (
        "row_ptr", "col_idx", "col_ptr", "row_idx", "groups", "meta")]


_vp, _i, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_s4 = ctypes.POINTER(ctypes.c_int64)

# name -> argument types; every function returns int except bsa_strerror
SIGNATURES = {
    "bsa_version": [],
    "bsa_strerror": [_i],
    "bsa_mask_reduce": [_vp, _s4, _i, _i, _i, _vp, _vp, _i, _vp],
    "bsa_tile_list_sizes": [_i, _i, _i, ctypes.POINTER(ListSizes)],
    "bsa_tile_lists_build": [_vp, _s4, _i, _i, _i] + [_vp] * 6 + [_vp],
    "bsa_attn_fwd": [_vp, _s4, _vp, _s4, _vp, _s4, _vp, _s4, _vp, _vp, _vp, _vp, _i, _i, _f, _i,
                     _i, _i, _i, _i, _vp, _vp, _vp],
    "bsa_attn_fwd_block_mask": [_vp, _s4, _vp, _s4, _vp, _s4, _vp, _s4, _vp, _vp, _vp, _s4, _i, _i,
                                _f, _i, _i, _i, _i, _i, _vp, _vp, _vp],
    "bsa_attn_fwd_rows": [_vp, _s4, _vp, _s4, _vp, _s4, _vp, _s4, _vp, _vp, _vp, _vp, _i, _i, _f, _i,
                          _i, _i, _i, _i, _i, _i, _vp, _s4, _vp, _vp, _vp],
    "bsa_attn_fwd_block_mask_rows": [_vp, _s4, _vp, _s4, _vp, _s4, _vp, _s4, _vp, _vp, _vp, _s4, _i,
                                     _i, _f, _i, _i, _i, _i, _i, _i, _i, _vp, _s4, _vp, _vp, _vp],
    "bsa_attn_bwd_delta": [_vp, _vp, _s4, _vp, _i, _i, _i, _i, _i, _vp],
    "bsa_attn_bwd_dkdv": [_vp, _vp, _vp, _vp, _s4, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i,
                          _i, _i, _i, _i, _vp, _s4, _vp, _vp, _vp],
    "bsa_attn_bwd_dq": [_vp, _vp, _vp, _vp, _s4, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i,
                        _i, _i, _i, _i, _vp, _s4, _vp, _vp, _vp],
    "bsa_reorder": [_vp, _vp, _s4, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "bsa_inv_reorder": [_vp, _vp, _s4, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "bsa_reorder_strided": [_vp, _s4, _vp, _s4, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "bsa_inv_reorder_strided": [_vp, _s4, _vp, _s4, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "bsa_attn_fwd_block_mask_static": [_vp, _s4, _vp, _s4, _vp, _s4, _vp, _s4, _vp, _vp, _s4, _i,
                                       _i, _f, _i, _i, _i, _i, _i, _vp],
    "bsa_static_warmup": [],
    "bsa_check_status": [_vp, _vp],
    "bsa_selftest_bounded_wait": [_vp, _vp, _vp],
}


def load():
    """Loads the library once; raises if it has not been built (run build.py next to csrc/)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python build.py` in the package directory; "
            "there is no fallback path")
    lib = ctypes.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = ctypes.c_char_p if name == "bsa_strerror" else ctypes.c_int
    _lib = lib
    return lib


def check(fn: str, status: int):
    if status != 0:
        raise BsaError(fn, status, load().bsa_strerror(status).decode())


def strides4(t: torch.Tensor):
    assert t.dim() == 4
    return (ctypes.c_int64 * 4)(*t.stride())


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_ptr(device=None):
    """The current stream of `device` as a cudaStream_t."""
    idx = -1 if device is None or device.index is None else device.index
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(idx))


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float16:
        return BSA_F16
    if dt == torch.bfloat16:
        return BSA_BF16
    raise TypeError(f"q, k, v must be float16 or bfloat16, got {dt}")
