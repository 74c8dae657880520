"""Compiling the CUDA sources of this folder for sm_100a and loading them.

Each `.cu` file becomes one shared library, built with nvcc directly (no torch
headers, so a file compiles in seconds) and loaded with ctypes. A library is
built the first time something needs it, or when its source, a header or the
flags changed; a line is printed to stderr when a compilation starts and ends,
so a first call on a fresh checkout shows what it is waiting for. Libraries go
to `csrc/_build/` inside the package; if that folder cannot be written, to a
per-user folder under the system's temporary directory.

There is no fallback: without nvcc or without a GPU the kernels do not exist
and every op fails with a clear error.
"""

from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared"]

#: library name -> its source file; every library is independent of the others
LIBRARIES = {
    "elementwise": "elementwise.cu",
    "norm": "norm.cu",
    "rope": "rope.cu",
    "attention_plain": "attention_plain.cu",
    "gemm_f32": "gemm_f32.cu",
    "sampling": "sampling.cu",
    "attention_decode": "attention_decode.cu",
    "attention_prefill": "attention_prefill.cu",
    "attention_prefill_tc": "attention_prefill_tc.cu",
    "gemm_tc": "gemm_tc.cu",
    "gemm_wide": "gemm_wide.cu",
    "gemm_pair": "gemm_pair.cu",
    "gemm_lib": "gemm_lib.cu",
}

#: extra flags of single libraries (libraries that need the driver API, for instance)
EXTRA_FLAGS: dict[str, list[str]] = {"gemm_lib": ["-lcublas"]}


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isfile(found):
        raise BuildError("nvcc was not found (looked on PATH and in /usr/local/cuda/bin): the "
                         "CUDA kernels of this library cannot be built, and there is no "
                         "other implementation to fall back to")
    return found


_dir_lock = threading.Lock()
_dir: Path | None = None


def _build_dir() -> Path:
    """Decided once per process (several threads may ask at the same time)."""
    global _dir
    with _dir_lock:
        if _dir is None:
            preferred = HERE / "_build"
            try:
                preferred.mkdir(exist_ok=True)
                probe = preferred / f".write_probe_{os.getpid()}_{threading.get_ident()}"
                probe.write_text("")
                probe.unlink()
                _dir = preferred
            except OSError:
                _dir = Path(tempfile.gettempdir()) / f"sakv_b200_build_{os.getuid()}"
                _dir.mkdir(parents=True, exist_ok=True)
        return _dir


def _headers() -> list[Path]:
    return sorted(HERE.glob("*.cuh")) + sorted(HERE.glob("*.h"))


def _fingerprint(name: str) -> str:
    h = hashlib.sha256()
    for path in [HERE / LIBRARIES[name]] + _headers():
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + EXTRA_FLAGS.get(name, [])).encode())
    return h.hexdigest()


def library_path(name: str) -> Path:
    return _build_dir() / f"libsakv_{name}.so"


def is_built(name: str) -> bool:
    out = library_path(name)
    stamp = out.with_suffix(".hash")
    return out.is_file() and stamp.is_file() and stamp.read_text() == _fingerprint(name)


def build(name: str, verbose: bool = True) -> Path:
    """Compile library `name` if it is missing or stale; returns its path."""
    if name not in LIBRARIES:
        raise BuildError(f"no library named {name!r}; known: {', '.join(sorted(LIBRARIES))}")
    out = library_path(name)
    if is_built(name):
        return out
    lock_path = out.with_suffix(".lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if is_built(name):          # another process built it while we waited
                return out
            src = HERE / LIBRARIES[name]
            tmp = out.with_suffix(f".tmp{os.getpid()}.so")
            cmd = ([_nvcc()] + ARCH_FLAGS + NVCC_FLAGS + EXTRA_FLAGS.get(name, [])
                   + ["-I", str(HERE), "-o", str(tmp), str(src)])
            if verbose:
                print(f"[build] compiling {src.name} for sm_100a ...", file=sys.stderr, flush=True)
            began = time.time()
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                    text=True)
            while True:
                try:
                    output, _ = proc.communicate(timeout=20)
                    break
                except subprocess.TimeoutExpired:
                    if verbose:
                        print(f"[build] ... still compiling {src.name} "
                              f"({time.time() - began:.0f} s)", file=sys.stderr, flush=True)
            if proc.returncode != 0:
                tmp.unlink(missing_ok=True)
                raise BuildError(f"nvcc failed on {src.name}:\n{output}")
            os.replace(tmp, out)
            out.with_suffix(".hash").write_text(_fingerprint(name))
            if verbose:
                print(f"[build] {src.name} done in {time.time() - began:.1f} s",
                      file=sys.stderr, flush=True)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return out


def build_all(verbose: bool = True, jobs: int | None = None) -> None:
    """Compile every library (several at a time)."""
    from concurrent.futures import ThreadPoolExecutor
    names = [n for n in LIBRARIES if not is_built(n)]
    if not names:
        return
    with ThreadPoolExecutor(max_workers=jobs or min(8, len(names))) as pool:
        for result in pool.map(lambda n: build(n, verbose), names):
            pass


_loaded: dict[str, ctypes.CDLL] = {}


def load(name: str) -> ctypes.CDLL:
    """The library, built if need be and loaded once per process."""
    lib = _loaded.get(name)
    if lib is None:
        lib = ctypes.CDLL(str(build(name)))
        _loaded[name] = lib
    return lib
