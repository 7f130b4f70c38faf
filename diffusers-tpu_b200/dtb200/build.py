"""Builds ``libdtb200_attn.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

Run ``python -m dtb200.build`` or call :func:`build`.  The library is rebuilt only
when a source under ``csrc/`` or the public header is newer than the binary.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC_DIR = os.path.join(os.path.dirname(PKG_DIR), "csrc")
INCLUDE_DIR = os.path.join(os.path.dirname(os.path.dirname(PKG_DIR)), "include")
LIB_PATH = os.path.join(PKG_DIR, "libdtb200_attn.so")

SOURCES = ["host_common.cu", "selftest.cu", "attn_api.cu", "prepass.cu", "smooth_k.cu", "out_proj.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
    "-cudart", "static",
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libdtb200_attn.so")


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR)]
    deps += [os.path.join(INCLUDE_DIR, f) for f in os.listdir(INCLUDE_DIR)]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False, extra_flags=(), out_path: str = LIB_PATH) -> str:
    """Compiles the library if needed and returns its path.

    ``extra_flags`` / ``out_path`` build an experimental variant beside the default binary
    (select it at load time with the ``DTB200_LIB`` environment variable)."""
    if out_path == LIB_PATH and not force and not _stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, *extra_flags]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC_DIR, s) for s in SOURCES]
    cmd += ["-o", out_path]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        sys.stderr.write(proc.stderr)
    return out_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
