"""Compiling the CUDA sources of `csrc/` for sm_100a and loading them.

Each `.cu` file becomes one shared library, built with nvcc the first time one of
its kernels is asked for and kept beside the sources in `csrc/_build/` under a name
that carries a hash of the sources and flags, so a stale library is never loaded.
The functions are plain `extern "C"` launchers and are called through ctypes with
raw device pointers and a stream; nothing links against torch, which keeps a
build to seconds per file.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise KernelBuildError("nvcc not found: the CUDA kernels cannot be built (set NVCC or put nvcc on PATH)")


def _sources_hash(name: str, extra_flags: list[str]) -> str:
    h = hashlib.sha256()
    for path in [CSRC / f"{name}.cu", *sorted(CSRC.glob("*.cuh")), *sorted(CSRC.glob("*.h"))]:
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + extra_flags).encode())
    return h.hexdigest()[:16]


_dir: Path | None = None
_dir_lock = threading.Lock()


def _build_dir() -> Path:
    """csrc/_build when it can be written, else a per-user folder under the temp dir."""
    global _dir
    with _dir_lock:
        if _dir is None:
            d = CSRC / "_build"
            try:
                d.mkdir(exist_ok=True)
                with tempfile.NamedTemporaryFile(dir=d, prefix=".probe"):
                    pass
            except OSError:
                d = Path(tempfile.gettempdir()) / f"longbow_quarrel_b200_build_{os.getuid()}"
                d.mkdir(exist_ok=True)
            _dir = d
        return _dir


def library_path(name: str, extra_flags: list[str] | None = None) -> Path:
    return _build_dir() / f"{name}.{_sources_hash(name, extra_flags or [])}.so"


def build(name: str, extra_flags: list[str] | None = None, verbose: bool = True) -> Path:
    """Compile csrc/<name>.cu if its library is not there yet; returns the .so path."""
    extra_flags = extra_flags or []
    src = CSRC / f"{name}.cu"
    if not src.is_file():
        raise KernelBuildError(f"no kernel source {src}")
    out = library_path(name, extra_flags)
    if out.is_file():
        return out
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [_nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, *extra_flags, "-I", str(CSRC), "-o", str(tmp), str(src)]
    if verbose:
        print(f"[longbow-quarrel_b200] compiling {src.name} for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def _tick():
        while not done.wait(10.0):
            if verbose:
                print(f"[longbow-quarrel_b200] still compiling {src.name} ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)
    ticker = threading.Thread(target=_tick, daemon=True)
    ticker.start()
    log, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise KernelBuildError(f"nvcc failed on {src.name}:\n{' '.join(cmd)}\n{log}")
    os.replace(tmp, out)
    for old in out.parent.glob(f"{name}.*.so"):
        if old != out and ".tmp" not in old.name:
            old.unlink(missing_ok=True)
    if verbose:
        print(f"[longbow-quarrel_b200] built {out.name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def load(name: str, extra_flags: list[str] | None = None) -> ctypes.CDLL:
    with _lock:
        if name not in _loaded:
            _loaded[name] = ctypes.CDLL(str(build(name, extra_flags)))
        return _loaded[name]


def all_sources() -> list[str]:
    return sorted(p.stem for p in CSRC.glob("*.cu"))


def build_all(verbose: bool = True) -> list[Path]:
    """Compile every kernel file (several at a time)."""
    from concurrent.futures import ThreadPoolExecutor
    names = all_sources()
    with ThreadPoolExecutor(max_workers=min(4, len(names) or 1)) as pool:
        return list(pool.map(lambda n: build(n, verbose=verbose), names))
