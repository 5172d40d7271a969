"""Compiles the CUDA sources under `csrc/` into one shared library for sm_100a.

The library has a plain C interface (no Python or torch headers), so each file
compiles in seconds and the result can be loaded by any caller. It is built in
tree (`cuca_b200/_build/`) when that folder can be written, else under the
temporary folder; a manifest of source hashes decides what is recompiled. The
first call in a fresh checkout compiles everything and prints a line per file.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
LIB_NAME = "libcuca_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"] + ARCH_FLAGS


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[cuca_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("CUCA_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise BuildError("nvcc was not found (looked at $CUCA_NVCC, PATH and /usr/local/cuda/bin): the CUDA "
                     "kernels of cuca_b200 cannot be compiled, and there is no fallback without them")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers_hash() -> str:
    h = hashlib.sha1()
    for p in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _writable(d: Path) -> bool:
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".probe-{os.getpid()}"
        probe.write_text("x")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    env = os.environ.get("CUCA_BUILD_DIR")
    if env:
        d = Path(env)
        if not _writable(d):
            raise BuildError(f"$CUCA_BUILD_DIR={env} cannot be written")
        return d
    in_tree = Path(__file__).resolve().parent.parent / "_build"
    if _writable(in_tree):
        return in_tree
    d = Path(tempfile.gettempdir()) / f"cuca_b200_build_{os.getuid()}"
    if not _writable(d):
        raise BuildError(f"neither {in_tree} nor {d} can be written: nowhere to build the kernels")
    return d


def _compile_one(nvcc: str, src: Path, obj: Path, log: Path) -> tuple[Path, float]:
    t0 = time.time()
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    log.write_text(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise BuildError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
    return src, time.time() - t0


class _BuildLock:
    """One builder at a time per build folder, across processes (two programs started together in a fresh checkout
    would otherwise write the same object files at once)."""

    def __init__(self, d: Path, verbose: bool):
        self.path, self.verbose, self.f = d / ".build.lock", verbose, None

    def __enter__(self):
        import fcntl
        self.f = open(self.path, "w")
        try:
            fcntl.flock(self.f, fcntl.LOCK_EX | fcntl.LOCK_NB)
        except OSError:
            if self.verbose:
                _say("another process is building the kernel library; waiting for it")
            fcntl.flock(self.f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *exc):
        import fcntl
        fcntl.flock(self.f, fcntl.LOCK_UN)
        self.f.close()


def build(verbose: bool = True, force: bool = False) -> Path:
    """Bring the library up to date and return its path."""
    d = build_dir()
    lib = _up_to_date(d) if not force else None
    if lib is not None:
        return lib
    with _BuildLock(d, verbose):
        return _build_locked(d, verbose, force)


def _up_to_date(d: Path):
    """The library's path if every source's hash is the one it was built from, else None."""
    lib = d / LIB_NAME
    try:
        manifest = json.loads((d / "manifest.json").read_text())
    except (OSError, ValueError):
        return None
    hh = _headers_hash()
    srcs = sources()
    if not srcs or not lib.is_file() or set(manifest) != {s.name for s in srcs}:
        return None
    for s in srcs:
        if manifest.get(s.name) != hashlib.sha1(s.read_bytes()).hexdigest() + hh:
            return None
    return lib


def _build_locked(d: Path, verbose: bool, force: bool) -> Path:
    lib = d / LIB_NAME
    manifest_path = d / "manifest.json"
    try:
        manifest = json.loads(manifest_path.read_text())
    except (OSError, ValueError):
        manifest = {}
    hh = _headers_hash()
    srcs = sources()
    if not srcs:
        raise BuildError(f"no CUDA sources under {CSRC}")
    todo = []
    new_manifest = {}
    for s in srcs:
        key = hashlib.sha1(s.read_bytes()).hexdigest() + hh
        new_manifest[s.name] = key
        obj = d / (s.stem + ".o")
        if force or manifest.get(s.name) != key or not obj.is_file():
            todo.append((s, obj))
    stale_lib = not lib.is_file() or set(manifest) != set(new_manifest)
    if not todo and not stale_lib:
        return lib
    nvcc = find_nvcc()
    if todo:
        if verbose:
            _say(f"compiling {len(todo)} CUDA source file(s) for sm_100a into {d} (first use; takes a minute or two)")
        t0 = time.time()
        workers = max(1, min(len(todo), os.cpu_count() or 2))
        with ThreadPoolExecutor(max_workers=workers) as pool:
            futs = [pool.submit(_compile_one, nvcc, s, o, d / (s.stem + ".log")) for s, o in todo]
            pending = set(futs)
            done_n = 0
            while pending:
                finished = {f for f in pending if f.done()}
                for f in finished:
                    src, dt = f.result()
                    done_n += 1
                    if verbose:
                        _say(f"  [{done_n}/{len(todo)}] {src.name} ({dt:.0f} s)")
                pending -= finished
                if pending:
                    time.sleep(0.5)
                    if verbose and int(time.time() - t0) % 15 == 0 and time.time() - t0 > 1:
                        _say(f"  still compiling, {len(pending)} file(s) left, {time.time() - t0:.0f} s so far")
                        time.sleep(1.0)
    objs = [str(d / (s.stem + ".o")) for s in srcs]
    tmp = d / (LIB_NAME + f".tmp{os.getpid()}")
    r = subprocess.run([nvcc, "-shared", *ARCH_FLAGS, "-o", str(tmp), *objs], capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    manifest_path.write_text(json.dumps(new_manifest, indent=1))
    if verbose:
        _say(f"built {lib}")
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
