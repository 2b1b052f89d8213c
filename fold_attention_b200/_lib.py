"""ctypes binding of libfold_b200.so, the C-ABI CUDA library behind the package.

There is no fallback: if the library is missing the import fails with the
command that builds it. Functions take raw device pointers
(`tensor.data_ptr()`), sizes and the current stream's handle.
"""

from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfold_b200.so")

P, I, F, Z, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t, ctypes.c_int64

# name -> argument types; every function returns int unless listed in _RESTYPES
_SIGNATURES = {
    "fold_abi_version": [],
    "fold_cache_write_prompt": [P, P, I, P, I, I, P, I, I, I, I, P, P, P, P, P, P, P, P, F, F, P],
    "fold_step_append": [P, P, P, I, I, I, I, I, P, I, I, P, P, P, P, P, P, P, P, P, P, F, P, P, P],
    "fold_tail_append": [P, I, I, I, I, P, I, I, P, I, P, P, P, P, P, P, P, I, P],
}
_RESTYPES = {"fold_last_error": ctypes.c_char_p}


class FoldLibraryError(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python fold_attention_b200/build.py` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    lib.fold_last_error.restype = ctypes.c_char_p
    lib.fold_last_error.argtypes = []
    for name, args in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = _RESTYPES.get(name, ctypes.c_int)
    return lib


def register(name, argtypes, restype=ctypes.c_int):
    """Declare one more entry point's signature (used by the submodules that
    own it)."""
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = restype
    _SIGNATURES[name] = argtypes


lib = _load()

_ERRORS = {1: ValueError, 4: NotImplementedError}


def call(name, *args):
    """Call an int-returning entry point; raise with the library's message on
    a non-zero status (bad argument -> ValueError, unsupported ->
    NotImplementedError, anything else -> FoldLibraryError)."""
    rc = getattr(lib, name)(*args)
    if rc != 0:
        msg = lib.fold_last_error().decode()
        raise _ERRORS.get(rc, FoldLibraryError)(f"{name}: {msg} (status {rc})")


def ptr(t):
    """A tensor's device address, or NULL for None."""
    return None if t is None else t.data_ptr()


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream(device):
    """The current torch stream of `device` as an integer handle."""
    ix = device.index if device.index is not None else torch.cuda.current_device()
    if _RAW_STREAM is not None:
        return _RAW_STREAM(ix)
    return torch.cuda.current_stream(ix).cuda_stream


def exported_symbols():
    """Every `fold_*` symbol the header declares, for the ABI test."""
    return sorted(list(_SIGNATURES) + ["fold_last_error"])
