"""Loads the compiled kernel library and declares its C functions.

There is no fallback: if the library cannot be built or loaded, or no CUDA
device is present, using a kernel raises `KernelLibraryError`.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_size_t, c_void_p

from . import build as _build


class KernelLibraryError(RuntimeError):
    pass


class KernelError(RuntimeError):
    """A kernel refused its arguments or failed to launch."""


_P = c_void_p
_I = c_int
_F = c_float

# name -> argument types (all return int)
_SIGNATURES = {
    "cuca_embed": [_P, _I, _P, _P, _I, _I, _I, _P, _P],
    "cuca_rmsnorm": [_P, _P, _I, _P, _I, _P, _I, _I, _F, _P],
    "cuca_rope_store": [_P, _I, _P, _P, _P, _I, _P, _P, _I, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "cuca_swiglu": [_P, _P, _I, _I, _I, _P],
    "cuca_add_to_stream": [_P, _P, _I, c_size_t, _P],
    "cuca_gemm_simt": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "cuca_attention_generic": [_P, _I, _P, _I, _I, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P, _P],
    "cuca_argmax": [_P, c_size_t, _I, _I, _P, _P],
    "cuca_suppress_tokens": [_P, c_size_t, _I, _I, _P, _I, _P],
    "cuca_scatter_int": [_P, _P, _P, _I, ctypes.c_longlong, _P],
    "cuca_sample": [_P, c_size_t, _I, _I, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _I, _P],
    "cuca_sample_max_split": [],
    "cuca_attention_max_head_dim": [],
    "cuca_attention_mma_supported": [_I, _I, _I, _I, _I],
    "cuca_attention_decode": [_P, _I, _P, _I, _P, _P, _I, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _F, _I, _I, _I,
                              _P, _P, _P, _P],
    "cuca_attention_decode_fused": [_P, _I, c_size_t, _P, _P, _P, _I, _I, _I, _P, _I, _P, _P, _I, _I, _P, _P, _P, _I,
                                    _P, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P, _P, _P],
    "cuca_attention_prefill": [_P, _I, _P, _I, _P, _P, _I, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _F, _I, _P,
                               _P],
    "cuca_decode_advance": [_P, _P, _P, _P, _P, _P, _I, _I, _P, _P, _P],
    "cuca_set_pdl": [_I],
    "cuca_attention_tc_supported": [_I, _I, _I, _I, _I, _I, _P, _P, _P],
    "cuca_attention_prefill_tc": [_P, _I, _I, _P, _I, _P, _P, _I, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _F, _I,
                                  _P, _P],
    "cuca_gemm_tc_partial_slices": [_I, _I, _I, _I],
    "cuca_gemm_tc_partial": [_P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P],
    "cuca_add_partials_rmsnorm": [_P, _P, _I, c_size_t, _P, _P, _I, _P, _I, _I, _F, _P],
    "cuca_add_partials": [_P, _P, _I, c_size_t, c_size_t, _P],
    "cuca_rope_store_partial": [_P, _I, c_size_t, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _P, _P, _I, _I, _I, _I,
                                _I, _I, _P, _P],
    "cuca_sm_count": [],
    "cuca_gemm_tc_partial_max_tokens": [],
    "cuca_gemm_pair_mode": [_I],
    "cuca_attention_pair_tiles_mode": [_I],
    "cuca_gemm_tc_partial_rows": [_I, _I],
    "cuca_wait_probe": [ctypes.c_ulonglong, _P, _P, _P],
    "cuca_attention_tile_rows": [_I],
    "cuca_attention_plan": [_P, _P, _P, _I, _I, _P, _I, _P, _P, _I, _P],
    "cuca_random_normal": [_P, _I, c_size_t, c_size_t, ctypes.c_ulonglong, _F, _F, _P],
    "cuca_gemm_tc_supported": [_P, _P, _I, _I, _I, _I],
    "cuca_gemm_tc": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, c_size_t, _P, _I, _I, _P, _P],
}

_lock = threading.Lock()
_lib = None


def load(verbose: bool = True):
    """Build (if needed) and load the library; cached after the first call."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        try:
            path = _build.build(verbose=verbose)
        except _build.BuildError as e:
            raise KernelLibraryError(f"the CUDA kernel library of cuca_b200 could not be built: {e}") from e
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelLibraryError(f"the CUDA kernel library {path} could not be loaded: {e}") from e
        lib.cuca_last_error.restype = ctypes.c_char_p
        lib.cuca_last_error.argtypes = []
        for name, args in _SIGNATURES.items():
            try:
                fn = getattr(lib, name)
            except AttributeError as e:
                raise KernelLibraryError(f"{path} lacks `{name}`: stale build? remove {path.parent}") from e
            fn.restype = c_int
            fn.argtypes = args
        _lib = lib
        return lib


def declare(name: str, argtypes: list) -> None:
    """Declare a further exported function (used by kernels added later in this package)."""
    _SIGNATURES[name] = argtypes
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.restype = c_int
        fn.argtypes = argtypes


launches = 0  # kernels launched through this library by this process (bench.py reports it)


def check(code: int, what: str) -> None:
    global launches
    launches += 1
    if code != 0:
        msg = _lib.cuca_last_error().decode(errors="replace") if _lib is not None else ""
        raise KernelError(f"{what}: {msg or 'error ' + str(code)}")
