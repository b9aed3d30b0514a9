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
HEADERS = ["common.cuh", "attention_tc_static.h", "tc5_common.cuh"]

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


def _with_global(defines):
    """A library's definitions plus the one that the environment asks of every library:
    KLLM_B200_TIMELINE=1 builds the instrumented variants (see common.cuh)."""
    d = dict(defines or {})
    if os.environ.get("KLLM_B200_TIMELINE", "0") not in ("", "0"):
        d["KLLM_TIMELINE"] = 1
    return d


def _define_flags(defines) -> List[str]:
    return [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]


def _variant(name: str, defines) -> str:
    """File stem of a library: the source name plus its compile-time definitions."""
    return name + "".join(f"-{k}{v}" for k, v in sorted((defines or {}).items()))


def _digest(name: str, defines=None) -> str:
    h = hashlib.sha256()
    for f in [name + ".cu"] + HEADERS:
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS + _define_flags(defines)).encode())
    return h.hexdigest()[:16]


def _find_built(name: str, digest: str):
    """A built library for these sources, in any of the folders a build may go to."""
    fname = f"{name}-{digest}.so"
    for d in (os.environ.get("KLLM_B200_BUILD_DIR"), os.path.join(CSRC, "_build"),
              os.path.join(tempfile.gettempdir(), f"kllm_b200-build-{os.getuid()}")):
        if d and os.path.isfile(os.path.join(d, fname)):
            return os.path.join(d, fname)
    return None


def compile_library(name: str, verbose: bool = True, defines=None) -> str:
    """Compile ``<name>.cu`` (with ``-D`` definitions, if any) unless a current
    build exists; return the .so path."""
    defines = _with_global(defines)
    src = os.path.join(CSRC, name + ".cu")
    if not os.path.isfile(src):
        raise KernelBuildError(f"kernel source {src} is missing")
    digest = _digest(name, defines)
    name_v = _variant(name, defines)
    built = _find_built(name_v, digest)
    if built:
        return built
    out_dir = build_dir()
    out = os.path.join(out_dir, f"{name_v}-{digest}.so")
    tmp = out + f".tmp{os.getpid()}"
    cmd = [find_nvcc()] + NVCC_FLAGS + _define_flags(defines) + ["-I", CSRC, "-o", tmp, src]
    if verbose:
        print(f"[kllm_b200] compiling {name_v} ({name}.cu) for sm_100a (first use) ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def _tick():
        while not done.wait(10.0):
            if verbose:
                print(f"[kllm_b200] ... still compiling {name_v} ({time.time() - t0:.0f} s)",
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
        raise KernelBuildError(f"nvcc failed for {name_v} (exit {proc.returncode}):\n{log}")
    os.replace(tmp, out)
    stale = len(name_v) + 1 + 16 + 3          # "<variant>-<16 hex>.so": builds of older sources
    for f in os.listdir(out_dir):
        if f.startswith(name_v + "-") and f.endswith(".so") and len(f) == stale and f != os.path.basename(out):
            try:
                os.unlink(os.path.join(out_dir, f))
            except OSError:
                pass
    if verbose:
        print(f"[kllm_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s",
              file=sys.stderr, flush=True)
    return out


def entry_arity(name: str) -> Dict[str, int]:
    """Number of parameters of every ``extern "C"`` function that ``<name>.cu`` defines,
    read from the source text."""
    import re
    with open(os.path.join(CSRC, name + ".cu")) as fh:
        text = re.sub(r"//[^\n]*", "", fh.read())
    out = {}
    for m in re.finditer(r'extern\s+"C"\s+[\w\s\*]+?\b(kllm_\w+)\s*\(([^)]*)\)\s*\{', text):
        params = m.group(2).strip()
        out[m.group(1)] = 0 if params in ("", "void") else params.count(",") + 1
    return out


class CheckedLibrary:
    """A loaded kernel library whose entry points refuse a call with another number
    of arguments than the C source declares: ctypes itself would pass whatever it is
    given, and the launcher would read the rest from wherever."""

    def __init__(self, cdll: ctypes.CDLL, arity: Dict[str, int], path: str):
        self._cdll, self._arity, self.path = cdll, arity, path

    def __getattr__(self, fname):
        fn = getattr(self._cdll, fname)
        want = self._arity.get(fname)
        if want is None:
            return fn

        def call(*args):
            if len(args) != want:
                raise KernelBuildError(f"{fname} takes {want} arguments, {len(args)} given")
            return fn(*args)
        call.__name__ = fname
        setattr(self, fname, call)
        return call


def load_library(name: str, defines=None) -> "CheckedLibrary":
    """The loaded library of ``<name>.cu`` (one per set of definitions), compiled
    now if needed."""
    key = _variant(name, _with_global(defines))
    lib = _loaded.get(key)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_library(name, defines=defines)
            try:
                lib = CheckedLibrary(ctypes.CDLL(path), entry_arity(name), path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
            _loaded[key] = lib
    return lib


def loaded_libraries() -> Dict[str, "CheckedLibrary"]:
    """Variant name -> library, for everything this process has loaded."""
    return dict(_loaded)


# Libraries that are built once per value of a compile-time size: build_all()
# compiles every allowed value, a running process only the one its model has.
VARIANTS = {"attention_tc": [{"KLLM_HD": hd} for hd in range(16, 129, 16)],
            "attention_tcgen05": [{"KLLM_HD": hd} for hd in (64, 128)],
            "attention_tcgen05_ptmem": [{"KLLM_HD": hd} for hd in (64, 128)]}


def build_all(verbose: bool = True) -> List[str]:
    out = []
    for n in sources():
        for defines in VARIANTS.get(n, [None]):
            out.append(compile_library(n, verbose=verbose, defines=defines))
    return out


if __name__ == "__main__":
    for p in build_all():
        print(p)
