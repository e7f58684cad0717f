"""Build the C-ABI shared library in-tree with nvcc (sm_100a only).

``python -m miniworld_engine_b200.build`` compiles ``csrc/trimul_api.cu`` (which
includes every kernel) into ``miniworld_engine_b200/libtrimul_b200.so``.  nvcc
cross-compiles without a GPU.  The library links the static CUDA runtime and
resolves the one driver symbol it needs at run time, so it has no link-time
dependency on libcuda and can be loaded next to PyTorch through ctypes.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_NAME = "libtrimul_b200.so"
LIB_PATH = os.path.join(PKG_DIR, LIB_NAME)

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-shared",
    "-cudart", "static",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the trimul_b200 library cannot be built")
    return nvcc


def sources() -> list[str]:  # microbench_sm100.cu is a separate program (build_microbench)
    return [os.path.join(CSRC, "trimul_api.cu")]


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(PKG_DIR), "include", "trimul_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False, extra: list[str] | None = None) -> str:
    """Compile the library if it is missing or older than its sources; return its path."""
    if not force and not needs_build():
        return LIB_PATH
    cmd = [find_nvcc(), *NVCC_FLAGS, *(extra or []), "-o", LIB_PATH, *sources()]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {res.returncode}")
    return LIB_PATH


def build_microbench(verbose: bool = True) -> str:
    """Compile ``csrc/microbench_sm100.cu`` (hardware micro-benchmarks behind the kernels' tile shapes)
    into ``miniworld_engine_b200/microbench_sm100``; it is not part of the library."""
    out = os.path.join(PKG_DIR, "microbench_sm100")
    cmd = [find_nvcc(), "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-o", out,
           os.path.join(CSRC, "microbench_sm100.cu")]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"nvcc failed with exit code {res.returncode}")
    return out


if __name__ == "__main__":
    if "--microbench" in sys.argv:
        print(build_microbench())
        sys.exit(0)
    print(build(force="--force" in sys.argv, verbose=True,
                extra=["-Xptxas", "-v"] if "--ptxas-v" in sys.argv else None))
