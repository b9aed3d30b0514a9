"""Builds the reference arm of bench.py: the reference's CUDA backend, unmodified.

    python baseline/build_reference.py PATH_TO_THE_REFERENCE_CHECKOUT

The reference is a Go program over one CUDA C++ backend (backend/model.cu, backend/shim.cu,
C ABI in backend/shim.h); its Go engine calls te_forward_batch once per step.  It has no
Python packaging and there is no Go toolchain here, so what is built is the backend
itself: its sources are copied as they are into baseline/_ref/backend/ (ignored by git)
and compiled with nvcc into baseline/_ref/libkllm_backend.so.  baseline/reference_arm.py
drives that library through the same C ABI the Go engine uses.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def main():
    if len(sys.argv) != 2 or not os.path.isdir(os.path.join(sys.argv[1], "backend")):
        print(__doc__)
        return 2
    src = os.path.join(sys.argv[1], "backend")
    dst = os.path.join(REF, "backend")
    os.makedirs(REF, exist_ok=True)
    if os.path.isdir(dst):
        os.chmod(dst, 0o755)
        shutil.rmtree(dst)
    os.makedirs(dst)
    for f in sorted(os.listdir(src)):                  # contents only: the checkout may be read-only
        if os.path.isfile(os.path.join(src, f)):
            shutil.copyfile(os.path.join(src, f), os.path.join(dst, f))
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    out = os.path.join(REF, "libkllm_backend.so")
    cus = sorted(os.path.join(dst, f) for f in os.listdir(dst) if f.endswith(".cu"))
    cmd = [nvcc, "-shared", "-O2", "-gencode", "arch=compute_100,code=sm_100", "-Xcompiler", "-fPIC",
           "-o", out] + cus + ["-lcublas"]
    print(" ".join(cmd))
    rc = subprocess.call(cmd)
    if rc == 0:
        print("built", out)
    return rc


if __name__ == "__main__":
    sys.exit(main())
