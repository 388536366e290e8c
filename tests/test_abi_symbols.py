"""The shared library builds for sm_100a, loads without a GPU and exports every symbol
that include/ue5m3_fp4.h declares.  No compute call is made here."""

from __future__ import annotations

import ctypes
import importlib.util
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _built_library() -> Path:
    spec = importlib.util.spec_from_file_location("ue5m3_build", ROOT / "ue5m3-fp4_b200" / "build.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module.build()


def _declared_symbols() -> list[str]:
    text = (ROOT / "include" / "ue5m3_fp4.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ue5m3_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(_built_library()))
    names = _declared_symbols()
    assert "ue5m3_quantize" in names and "ue5m3_gemm_issue_rz_bf16" in names and "ue5m3_amax" in names
    missing = [name for name in names if not hasattr(lib, name)]
    assert not missing, missing


def test_version_and_status_strings():
    lib = ctypes.CDLL(str(_built_library()))
    lib.ue5m3_status_string.restype = ctypes.c_char_p
    assert lib.ue5m3_abi_version() == 2
    assert lib.ue5m3_status_string(0) == b"ok"
    assert b"16 or 32" in lib.ue5m3_status_string(2)
    lib.ue5m3_amax_scratch_bytes.restype = ctypes.c_size_t
    assert 4096 <= lib.ue5m3_amax_scratch_bytes() <= 65536
    lib.ue5m3_window_record_ints.restype = ctypes.c_size_t
    lib.ue5m3_window_record_ints.argtypes = [ctypes.c_int64]
    assert lib.ue5m3_window_record_ints(300) == 4 + 4096 + 2 * 300


def test_argument_validation_needs_no_device():
    lib = ctypes.CDLL(str(_built_library()))
    p, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
    lib.ue5m3_quantize.argtypes = [p, i32, i64, i64, i32, i32, p, f32, i32, p, i32, p, p, p, p, p, p, i32, i32, p]
    fake = 0x1000
    args = dict(x=fake, dtype=0, rows=4, cols=64, block=16, blocking=0, amax=fake, target=448.0, rounding=0,
                bits=None, bits_dtype=0)
    def call(**over):
        a = {**args, **over}
        return lib.ue5m3_quantize(a["x"], a["dtype"], a["rows"], a["cols"], a["block"], a["blocking"], a["amax"],
                                  a["target"], a["rounding"], a["bits"], a["bits_dtype"], None, None, None, None,
                                  None, None, 0, 0, None)
    assert call(x=None) == 1
    assert call(block=64) == 2
    assert call(rounding=3) == 1
    assert call(rounding=7) == 1  # stochastic without bits
    assert call(bits=fake) == 1  # bits with ties-to-even
    assert call(target=0.0) == 1
    lib.ue5m3_gemm_issue_rz_bf16.argtypes = [p, p, i64, i64, i64, i32, p, p, p, f32, p, i32, p, i32, i64, p, p]
    assert lib.ue5m3_gemm_issue_rz_bf16(fake, fake, 8, 8, 65, 0, None, None, None, 0.0, None, 0, fake, 1, 8, None, None) == 3
    assert lib.ue5m3_gemm_issue_rz_bf16(fake + 2, fake, 8, 8, 64, 0, None, None, None, 0.0, None, 0, fake, 1, 8, None, None) == 4
    # alpha comes either as a ready scalar or as two amax scalars, never both, never one amax alone
    assert lib.ue5m3_gemm_issue_rz_bf16(fake, fake, 8, 8, 64, 0, fake, fake, fake, 1.0, None, 0, fake, 1, 8, None, None) == 1
    assert lib.ue5m3_gemm_issue_rz_bf16(fake, fake, 8, 8, 64, 0, None, fake, None, 1.0, None, 0, fake, 1, 8, None, None) == 1
