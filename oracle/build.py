"""Compile the C oracle into oracle/_build/libue5m3_oracle.so with gcc and, where the reference
checkout is present, place a copy of its Python package under the git-ignored oracle/_ref/ so
that the GPU parity tests can run the reference's own Triton kernels as a second oracle.

Test infrastructure only: the shipped package never loads either.
"""

from __future__ import annotations

import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCE = HERE / "ue5m3_oracle.c"
OUTPUT = HERE / "_build" / "libue5m3_oracle.so"
REFERENCE_PACKAGE = Path(os.environ.get("UE5M3_REFERENCE_ROOT", "/root/reference")) / "src" / "ue5m3_fp4"
REFERENCE_COPY = HERE / "_ref" / "src"


def place_reference_copy() -> Path | None:
    """oracle/_ref/src/ue5m3_fp4 = the reference's package, unmodified (never committed: the
    directory is git-ignored).  Returns None when no reference checkout is reachable."""

    import shutil

    if not (REFERENCE_PACKAGE / "backends" / "triton" / "api.py").exists():
        return REFERENCE_COPY if (REFERENCE_COPY / "ue5m3_fp4").exists() else None
    target = REFERENCE_COPY / "ue5m3_fp4"
    if target.exists():
        shutil.rmtree(target)
    shutil.copytree(REFERENCE_PACKAGE, target, ignore=shutil.ignore_patterns("__pycache__"))
    return REFERENCE_COPY


def build(force: bool = False) -> Path:
    place_reference_copy()
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
