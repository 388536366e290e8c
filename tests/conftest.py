"""Shared fixtures: import paths, the ``gpu`` marker and the golden fixtures."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
for entry in (ROOT, ROOT / "ue5m3-fp4_b200"):
    if str(entry) not in sys.path:
        sys.path.insert(0, str(entry))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def quantize_golden():
    return np.load(ROOT / "tests" / "golden" / "quantize_golden.npz")


@pytest.fixture(scope="session")
def gemm_golden():
    return np.load(ROOT / "tests" / "golden" / "gemm_golden.npz")


@pytest.fixture(scope="session")
def rht_golden():
    return np.load(ROOT / "tests" / "golden" / "rht_golden.npz")


def golden_case_names(npz) -> list[str]:
    return sorted({key.split(".")[0] for key in npz.files})


@pytest.fixture(params=["fp4", "bf16"])
def gemm_path(request, monkeypatch):
    """Run a test once per GEMM kernel: FP4 block-scaled tensor cores and the BF16-issue kernel."""

    monkeypatch.setenv("UE5M3_GEMM_PATH", request.param)
    return request.param
