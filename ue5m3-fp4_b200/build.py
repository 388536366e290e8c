"""Build the sm_100a shared library (CUDA kernels + C ABI) in-tree with nvcc.

    python ue5m3-fp4_b200/build.py

produces ue5m3-fp4_b200/lib/libue5m3_b200.so.  nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCES = ["abi.cu", "amax.cu", "quantize.cu", "quantize_operand.cu", "gemm_sm100.cu", "gemm_fp4_sm100.cu",
           "gemm_fallback.cu", "fallback_workspace.cu", "window_place.cu"]
OUTPUT = HERE / "lib" / "libue5m3_b200.so"


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    candidate = Path(cuda_home) / "bin" / "nvcc"
    return str(candidate) if candidate.exists() else "nvcc"


def build(force: bool = False, verbose: bool = False) -> Path:
    csrc = HERE / "csrc"
    deps = list(csrc.glob("*.cu")) + list(csrc.glob("*.cuh")) + [HERE.parent / "include" / "ue5m3_fp4.h"]
    newest = max(p.stat().st_mtime for p in deps)
    if not force and OUTPUT.exists() and OUTPUT.stat().st_mtime >= newest:
        return OUTPUT
    OUTPUT.parent.mkdir(exist_ok=True)
    objects = []
    commands = []
    for name in SOURCES:
        obj = OUTPUT.parent / (name + ".o")
        command = [
            _nvcc(), "-O3", "-std=c++17",
            "-gencode", "arch=compute_100a,code=sm_100a",
            "-lineinfo", "--fmad=false",
            "-Xcompiler", "-fPIC",
            "-c", str(csrc / name), "-o", str(obj),
        ]
        if verbose:
            command.insert(1, "-Xptxas")
            command.insert(2, "-v")
        commands.append(command)
        objects.append(str(obj))
    if verbose:  # keep each file's ptxas listing together
        for command in commands:
            subprocess.run(command, check=True)
    else:
        from concurrent.futures import ThreadPoolExecutor

        with ThreadPoolExecutor(max_workers=min(len(commands), os.cpu_count() or 1)) as pool:
            for done in pool.map(lambda c: subprocess.run(c, check=True), commands):
                done.check_returncode()
    subprocess.run(
        [_nvcc(), "-shared", "-o", str(OUTPUT), *objects, "-gencode", "arch=compute_100a,code=sm_100a"],
        check=True,
    )
    return OUTPUT


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
