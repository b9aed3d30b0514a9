"""Builds and loads the CUDA kernel libraries, one shared object per ``.cu`` file.

A library is compiled with nvcc for sm_100a the first time one of its kernels is
asked for, so a process compiles what its model needs and no more.  The shared
object is named after a hash of its sources and flags and kept beside the sources
(``csrc/_build/``), or in a per-user folder under the temporary directory when
the package folder is read-only.  There is no fallback: when nvcc or a source is
missing, or the compilation fails, ``KernelBuildError`` is raised.
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
from typing import Dict, List

CSRC = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-lineinfo", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
                           "--expt-relaxed-constexpr"]
HEADERS = ["common.cuh"]

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def sources() -> List[str]:
    """Names (without .cu) of every kernel library in this folder."""
    return sorted(f[:-3] for f in os.listdir(CSRC) if f.endswith(".cu"))


def find_nvcc() -> str:
    cands = [os.environ.get("KLLM_B200_NVCC"), shutil.which("nvcc")]
    for home in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if home:
            cands.append(os.path.join(home, "bin", "nvcc"))
    for c in cands:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise KernelBuildError("nvcc not found (PATH, CUDA_HOME, /usr/local/cuda): the CUDA kernels of "
                           "kllm_b200 cannot be built and there is no fallback path")


def build_dir() -> str:
    env = os.environ.get("KLLM_B200_BUILD_DIR")
    cands = [env] if env else []
    cands.append(os.path.join(CSRC, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"kllm_b200-build-{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.unlink(probe)
            return d
        except OSError:
            continue
    raise KernelBuildError(f"no writable build folder among {cands}")


def _digest(name: str) -> str:
    h = hashlib.sha256()
    for f in [name + ".cu"] + HEADERS:
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _find_built(name: str, digest: str):
    """A built library for these sources, in any of the folders a build may go to."""
    fname = f"{name}-{digest}.so"
    for d in (os.environ.get("KLLM_B200_BUILD_DIR"), os.path.join(CSRC, "_build"),
              os.path.join(tempfile.gettempdir(), f"kllm_b200-build-{os.getuid()}")):
        if d and os.path.isfile(os.path.join(d, fname)):
            return os.path.join(d, fname)
    return None


def compile_library(name: str, verbose: bool = True) -> str:
    """Compile ``<name>.cu`` if no current build exists; return the .so path."""
    src = os.path.join(CSRC, name + ".cu")
    if not os.path.isfile(src):
        raise KernelBuildError(f"kernel source {src} is missing")
    digest = _digest(name)
    built = _find_built(name, digest)
    if built:
        return built
    out_dir = build_dir()
    out = os.path.join(out_dir, f"{name}-{digest}.so")
    tmp = out + f".tmp{os.getpid()}"
    cmd = [find_nvcc()] + NVCC_FLAGS + ["-I", CSRC, "-o", tmp, src]
    if verbose:
        print(f"[kllm_b200] compiling {name}.cu for sm_100a (first use) ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def _tick():
        while not done.wait(10.0):
            if verbose:
                print(f"[kllm_b200] ... still compiling {name}.cu ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)

    ticker = threading.Thread(target=_tick, daemon=True)
    ticker.start()
    try:
        log, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed for {name}.cu (exit {proc.returncode}):\n{log}")
    os.replace(tmp, out)
    for f in os.listdir(out_dir):  # builds of older sources of the same library
        if f.startswith(name + "-") and f.endswith(".so") and f != os.path.basename(out):
            try:
                os.unlink(os.path.join(out_dir, f))
            except OSError:
                pass
    if verbose:
        print(f"[kllm_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s",
              file=sys.stderr, flush=True)
    return out


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library of ``<name>.cu``, compiled now if needed."""
    lib = _loaded.get(name)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
            _loaded[name] = lib
    return lib


def build_all(verbose: bool = True) -> List[str]:
    return [compile_library(n, verbose=verbose) for n in sources()]


if __name__ == "__main__":
    for p in build_all():
        print(p)
