"""Compile the C oracle into oracle/_build/libue5m3_oracle.so with gcc.

Test infrastructure only: the shipped package never loads this library.
"""

from __future__ import annotations

import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCE = HERE / "ue5m3_oracle.c"
OUTPUT = HERE / "_build" / "libue5m3_oracle.so"


def build(force: bool = False) -> Path:
    OUTPUT.parent.mkdir(exist_ok=True)
    if (
        not force
        and OUTPUT.exists()
        and OUTPUT.stat().st_mtime >= SOURCE.stat().st_mtime
    ):
        return OUTPUT
    compiler = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else os.environ.get("CC", "gcc")
    command = [
        compiler,
        "-O2",
        "-std=gnu11",
        "-fPIC",
        "-shared",
        "-fopenmp",
        "-ffp-contract=off",
        "-frounding-math",
        "-fno-fast-math",
        "-fexcess-precision=standard",
        "-msse2",
        "-mfpmath=sse",
        str(SOURCE),
        "-o",
        str(OUTPUT),
        "-lm",
    ]
    try:
        subprocess.run(command, check=True)
    except subprocess.CalledProcessError:
        # No OpenMP runtime for this compiler: build the same source single-threaded.
        subprocess.run([c for c in command if c != "-fopenmp"], check=True)
    return OUTPUT


if __name__ == "__main__":
    print(build(force=True))
