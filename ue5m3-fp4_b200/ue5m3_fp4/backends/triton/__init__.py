"""Entry points under the module path the reference's callers import.

The reference ships its quantizer and issue-RZ GEMM as Triton kernels in
``ue5m3_fp4.backends.triton`` (backends/triton/__init__.py:19-60) and
``nn/linear.py`` imports that path at call time.  The same four names are
kept here; they run the sm_100a CUDA kernels, not Triton.
"""

from __future__ import annotations


def triton_available() -> bool:
    """True when a CUDA device and the built sm_100a library are present."""

    from ue5m3_fp4.backends import b200

    return b200.available()


def fake_quantize_gemm_operands(*args, **kwargs):
    from ue5m3_fp4.backends import b200

    return b200.fake_quantize_gemm_operands(*args, **kwargs)


def issue_rz_bf16_gemm(*args, **kwargs):
    from ue5m3_fp4.backends import b200

    return b200.issue_rz_bf16_gemm(*args, **kwargs)


def probe_matched_fp4_gemm(*args, **kwargs):
    from ue5m3_fp4.backends import b200

    return b200.probe_matched_fp4_gemm(*args, **kwargs)


__all__ = [
    "fake_quantize_gemm_operands",
    "issue_rz_bf16_gemm",
    "probe_matched_fp4_gemm",
    "triton_available",
]
