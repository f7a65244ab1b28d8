"""Builds ``lib/libb200lora.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

``python -m nanovllm_voxcpm_b200.build`` or ``build_library()``.  nvcc cross-compiles
without a GPU.  The CUDA runtime is linked statically so the library loads next to any
torch build; nothing from torch is linked.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_DIR = os.path.join(_HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libb200lora.so")
#: the same library compiled with -DB200_LORA_DEBUG_BOUNDS: every index taken from caller metadata is checked on the
#: device and a violation is reported through the status word (load it with B200_LORA_LIB=<this path>)
DEBUG_LIB_PATH = os.path.join(LIB_DIR, "libb200lora_debug.so")
#: tuning build (-DB200_TRACE): the fused decode kernel records SM-clock timestamps of its phases, read back with
#: lora_b200_debug_trace; used by ``python -m nanovllm_voxcpm_b200.timeline``. Slower than the product build.
TRACE_LIB_PATH = os.path.join(LIB_DIR, "libb200lora_trace.so")
SOURCES = ["api.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "-cudart", "static",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the B200 LoRA library cannot be built")
    return exe


def _stale(path: str = LIB_PATH) -> bool:
    if not os.path.exists(path):
        return True
    built = os.path.getmtime(path)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(_HERE), "include", "b200_lora.h"))
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def build_library(force: bool = False, verbose: bool = False, debug_bounds: bool = False, trace: bool = False) -> str:
    target = TRACE_LIB_PATH if trace else DEBUG_LIB_PATH if debug_bounds else LIB_PATH
    if not force and not _stale(target):
        return target
    os.makedirs(LIB_DIR, exist_ok=True)
    defines = ["-DB200_TRACE"] if trace else ["-DB200_LORA_DEBUG_BOUNDS"] if debug_bounds else []
    cmd = [_nvcc(), *NVCC_FLAGS, *defines, "-o", target,
           *[os.path.join(CSRC, s) for s in SOURCES]]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        sys.stderr.write(proc.stderr)
    return target


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv, debug_bounds="--debug-bounds" in sys.argv,
                        trace="--trace" in sys.argv))
