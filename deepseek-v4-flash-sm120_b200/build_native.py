"""Build `deepseek_v4_kernel/libdsv4_b200.so` in-tree with nvcc for sm_100a.

    python build_native.py [--verbose] [--force]

The library is the C-ABI declared in include/dsv4_b200.h; it links the CUDA
runtime statically and depends on nothing else.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.environ.get("DSV4_BUILD_OUT") or os.path.join(HERE, "deepseek_v4_kernel", "libdsv4_b200.so")
SOURCES = ["capi.cu", "simple_kernels.cu", "umma_selftest.cu", "sparse_attn_sm100.cu",
           "noalloc_entry.cu", "head_gather.cu"]


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps += [os.path.join(ROOT, "include", "dsv4_b200.h"), os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and not _stale():
        return OUT
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-shared", "-Xcompiler", "-fPIC", "-I" + os.path.join(ROOT, "include"), "-I" + CSRC,
           "--threads", "4", "-diag-suppress", "177"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    if os.environ.get("DSV4_EXTRA_DEFINES"):
        cmd += ["-D" + d for d in os.environ["DSV4_EXTRA_DEFINES"].split(",")]
    if os.environ.get("DSV4_KERNEL_DEBUG"):
        cmd += ["-DDSV4_DEBUG=1"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES] + ["-o", OUT]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode:
        raise RuntimeError("nvcc failed building libdsv4_b200.so")
    return OUT


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force="--force" in sys.argv))
