"""The host core: cache bookkeeping, step packing and the scheduler's decisions, in C++ (`csrc/host/`).

It has a plain C interface and needs neither CUDA nor a GPU; `g++` compiles it into `libcuca_host.so` next to the
kernel library at first use (a manifest of source hashes decides when it is compiled again). The Python classes
in `cache/pages.py`, `engine/step.py` and `engine/scheduler.py` are thin wrappers around it.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import threading
from ctypes import POINTER, c_char_p, c_int, c_longlong, c_void_p
from pathlib import Path

from ..kernels.build import BuildError, _say, build_dir

SRC = Path(__file__).resolve().parent.parent / "csrc" / "host"
LIB_NAME = "libcuca_host.so"
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-shared"]

OK, EXHAUSTED, BOOKKEEPING, INVALID, TOO_SMALL = 0, 1, 2, 3, 4


class HostLibraryError(RuntimeError):
    """The host core could not be built or loaded."""


def _find_cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and shutil.which(cand):
            return cand
    raise BuildError("no C++ compiler was found (looked at $CXX, g++, c++, clang++): the host core of cuca_b200 "
                     "cannot be compiled")


def build(verbose: bool = True) -> Path:
    d = build_dir()
    lib = d / LIB_NAME
    stamp = d / "host.sha1"
    h = hashlib.sha1(" ".join(CXX_FLAGS).encode())
    files = sorted(SRC.glob("*.cpp")) + sorted(SRC.glob("*.hpp"))
    if not files:
        raise BuildError(f"no sources under {SRC}")
    for p in files:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    digest = h.hexdigest()
    try:
        if lib.is_file() and stamp.read_text() == digest:
            return lib
    except OSError:
        pass
    cxx = _find_cxx()
    if verbose:
        _say(f"compiling the host core ({len(files)} files) with {Path(cxx).name} into {d}")
    tmp = d / (LIB_NAME + f".tmp{os.getpid()}")
    cmd = [cxx, *CXX_FLAGS, "-o", str(tmp), *[str(p) for p in files if p.suffix == ".cpp"]]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"compiling the host core failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    stamp.write_text(digest)
    return lib


_I, _P, _L = c_int, c_void_p, c_longlong
_IP = POINTER(c_int)
# name -> (result type, argument types)
_SIGNATURES = {
    "cuca_host_blockpool_new": (_P, [_I]), "cuca_host_blockpool_free": (None, [_P]),
    "cuca_host_blockpool_alloc": (_I, [_P]), "cuca_host_blockpool_release": (_I, [_P, _I]),
    "cuca_host_blockpool_free_count": (_I, [_P]), "cuca_host_blockpool_reset": (None, [_P]),
    "cuca_host_pools_new": (_P, [_I, _IP, _IP, _I]), "cuca_host_pools_free": (None, [_P]),
    "cuca_host_pools_new_seq": (_I, [_P]), "cuca_host_pools_drop_seq": (None, [_P, _I]),
    "cuca_host_pools_owed": (None, [_P, _I, _I, _IP]), "cuca_host_pools_can_give": (_I, [_P, _IP]),
    "cuca_host_pools_reserve": (_I, [_P, _I, _I]), "cuca_host_pools_release_window": (_I, [_P, _I]),
    "cuca_host_pools_truncate": (_I, [_P, _I, _I]), "cuca_host_pools_release": (_I, [_P, _I]),
    "cuca_host_pools_publish": (_I, [_P, _I, _IP, _I]), "cuca_host_pools_finish": (_I, [_P, _I, _IP, _I]),
    "cuca_host_pools_new_seq_with_prefix": (_I, [_P, _IP, _I]), "cuca_host_pools_cached_blocks": (_I, [_P, _I]),
    "cuca_host_pools_reset": (None, [_P]), "cuca_host_pools_check": (_I, [_P]), "cuca_host_pools_live": (_I, [_P]),
    "cuca_host_pools_free_blocks": (_I, [_P, _I]), "cuca_host_pools_total_blocks": (_I, [_P, _I]),
    "cuca_host_seq_get": (_I, [_P, _I, _I]), "cuca_host_seq_set": (_I, [_P, _I, _I, _I]),
    "cuca_host_seq_table": (_I, [_P, _I, _I, _IP, _I]),
    "cuca_host_slots_new": (_P, [_I]), "cuca_host_slots_free": (None, [_P]), "cuca_host_slots_alloc": (_I, [_P]),
    "cuca_host_slots_release": (_I, [_P, _I]), "cuca_host_slots_free_count": (_I, [_P]),
    "cuca_host_slots_reset": (None, [_P]),
    "cuca_host_step_pack": (_I, [_P, _I, _IP, _IP, _IP, _IP, _IP, _IP, _I, _I, _I, _I, _P, _I, _IP, _IP]),
    "cuca_host_step_validate": (_I, [_P, _I, _IP, _IP, _IP, _IP, _I, _I, _I]),
    "cuca_host_table_updates": (_I, [_P, _IP, _IP, _I, _I, _I, _P, _I]),
    "cuca_host_step_advance": (_I, [_P, _IP, _IP, _I]),
    "cuca_host_sched_new": (_P, [_P, _P, _I, _I, _I, _I, _IP, _I, _I]), "cuca_host_sched_free": (None, [_P]),
    "cuca_host_sched_submit": (_I, [_P, _IP, _I, _L, _I, _IP, _I]), "cuca_host_sched_admit": (None, [_P]),
    "cuca_host_sched_plan": (_I, [_P, _IP, _I]), "cuca_host_sched_apply": (_I, [_P, _IP, _I]),
    "cuca_host_sched_fail_running": (None, [_P, c_char_p]), "cuca_host_sched_forget": (None, [_P, _I]), "cuca_host_sched_cancel": (None, [_P, _I]),
    "cuca_host_sched_events": (_I, [_P, _IP, _I]), "cuca_host_sched_counter": (_L, [_P, _I]),
    "cuca_host_sched_seq_get": (_L, [_P, _I, _I]), "cuca_host_sched_seq_error": (c_char_p, [_P, _I]),
    "cuca_host_sched_list": (_I, [_P, _I, _IP, _I]),
    "cuca_host_last_error": (c_char_p, []),
}

_lock = threading.Lock()
_lib = None


def load(verbose: bool = True):
    """Build (if needed) and load the host core; cached after the first call."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        try:
            path = build(verbose=verbose)
        except BuildError as e:
            raise HostLibraryError(f"the host core of cuca_b200 could not be built: {e}") from e
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise HostLibraryError(f"the host core {path} could not be loaded: {e}") from e
        for name, (res, args) in _SIGNATURES.items():
            try:
                fn = getattr(lib, name)
            except AttributeError as e:
                raise HostLibraryError(f"{path} lacks `{name}`: stale build? remove {path.parent}") from e
            fn.restype = res
            fn.argtypes = args
        _lib = lib
        return lib


def last_error() -> str:
    return (_lib.cuca_host_last_error() or b"").decode(errors="replace") if _lib is not None else ""


def ints(values) -> ctypes.Array:
    """A C array of ints from a Python sequence."""
    values = list(values)
    return (c_int * max(1, len(values)))(*values)
