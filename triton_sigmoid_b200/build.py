"""Builds the CUDA library of this package in-tree with nvcc (sm_100a only).

    python -m triton_sigmoid_b200.build [--force] [--verbose]

The result, ``triton_sigmoid_b200/lib/libsigattn_b200.so``, exports the C ABI declared in
``include/sigattn_b200.h``.  nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

from ._paths import CSRC, LIB_DIR, LIB_PATH, PKG_DIR, ROOT  # noqa: F401

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _sources():
    srcs = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC))]
    srcs.append(os.path.join(ROOT, "include", "sigattn_b200.h"))
    return srcs


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(s) > t for s in _sources())


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: set NVCC or put it on PATH")


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library (skipped when it is newer than its sources, unless `force`)."""
    target = LIB_PATH
    if not force and not needs_build():
        return LIB_PATH
    os.makedirs(os.path.dirname(target), exist_ok=True)
    cmd = [find_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", target, os.path.join(CSRC, "sigattn_api.cu")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building " + target)
    return target


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
