"""ctypes binding of the sm_100a shared library (the C ABI in include/ue5m3_fp4.h).

There is no fallback: if the library is missing, every operation raises.  PyTorch
is used only for device memory and streams; all arithmetic runs in the library.
"""

from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

UE5M3_OK = 0
DTYPE_BF16 = 0
DTYPE_FP32 = 1
ROUND_TIES_TO_EVEN = 0
ROUND_STOCHASTIC_FAST = 7
BITS_NONE = 0
BITS_U8 = 1
BITS_I32 = 2
BITS_PHILOX = 3
BLOCK_ROW = 0
BLOCK_COL = 1
BLOCK_2D = 2
FAKE_NONE = 0
FAKE_ENCODED = 1
FAKE_DECODED = 2
FAKE_DEQUANT = 3

_LIB_ENV = "UE5M3_FP4_B200_LIB"
_DEFAULT_LIB = Path(__file__).resolve().parent.parent / "lib" / "libue5m3_b200.so"

_lib: ctypes.CDLL | None = None


class NativeLibraryError(RuntimeError):
    """The sm_100a library is missing or returned an error status."""


def library_path() -> Path:
    return Path(os.environ.get(_LIB_ENV, str(_DEFAULT_LIB)))


def load() -> ctypes.CDLL:
    """Load the shared library once; fail loudly when it has not been built."""

    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        raise NativeLibraryError(
            f"the sm_100a library {path} does not exist; build it with "
            "`python ue5m3-fp4_b200/build.py` (there is no CPU or Triton fallback)"
        )
    lib = ctypes.CDLL(str(path))
    p, i32, i64, f32, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_size_t
    lib.ue5m3_abi_version.restype = i32
    lib.ue5m3_status_string.restype = ctypes.c_char_p
    lib.ue5m3_status_string.argtypes = [i32]
    lib.ue5m3_last_cuda_error.restype = ctypes.c_char_p
    lib.ue5m3_amax_scratch_bytes.restype = sz
    lib.ue5m3_amax.restype = i32
    lib.ue5m3_amax.argtypes = [p, i32, i64, p, p, sz, p]
    lib.ue5m3_quantize.restype = i32
    lib.ue5m3_quantize.argtypes = [p, i32, i64, i64, i32, i32, p, f32, i32, p, i32, p, p, p, p, p, p, i32, i32, p]
    lib.ue5m3_dequantize.restype = i32
    lib.ue5m3_dequantize.argtypes = [p, p, i64, i64, i32, i32, p, f32, p, i32, p]
    lib.ue5m3_alpha.restype = i32
    lib.ue5m3_alpha.argtypes = [p, p, f32, p, p]
    lib.ue5m3_gemm_issue_rz_bf16.restype = i32
    lib.ue5m3_gemm_issue_rz_bf16.argtypes = [p, p, i64, i64, i64, i32, p, p, p, f32, p, i32, p, i32, i64, p, p]
    lib.ue5m3_packed_scales_bytes.restype = sz
    lib.ue5m3_packed_scales_bytes.argtypes = [i64, i64]
    lib.ue5m3_pack_scales_ue4m3.restype = i32
    lib.ue5m3_pack_scales_ue4m3.argtypes = [p, i64, i64, i32, i32, i32, p, p, p, p]
    lib.ue5m3_window_record_ints.restype = sz
    lib.ue5m3_window_record_ints.argtypes = [i64]
    lib.ue5m3_quantize_fp4_operand.restype = i32
    lib.ue5m3_quantize_fp4_operand.argtypes = [p, i32, i64, i64, i32, i32, p, f32, i32, p, i32, i32, p, p, p, p, p, p]
    lib.ue5m3_quantize_fp4_operand_t.restype = i32
    lib.ue5m3_quantize_fp4_operand_t.argtypes = [p, i32, i64, i64, i32, i32, p, f32, i32, p, i32, i32, p, p, p, p, p]
    lib.ue5m3_rht_amax_t.restype = i32
    lib.ue5m3_rht_amax_t.argtypes = [p, i32, i64, i64, p, p]
    lib.ue5m3_quantize_fp4_operand_t_rht.restype = i32
    lib.ue5m3_quantize_fp4_operand_t_rht.argtypes = [p, i32, i64, i64, p, f32, i32, p, i32, i32, p, p, p, p, p]
    lib.ue5m3_gemm_fp4_fallback.restype = i32
    lib.ue5m3_gemm_fp4_fallback.argtypes = [p, p, p, p, p, p, i64, i64, i64, i32, p, p, p, f32, p, i32, p, i32, i64, p, p]
    lib.ue5m3_fallback_workspace_bytes.restype = ctypes.c_size_t
    lib.ue5m3_fallback_workspace_bytes.argtypes = [i64, i64, i64]
    lib.ue5m3_gemm_fp4_fallback_ws.restype = i32
    lib.ue5m3_gemm_fp4_fallback_ws.argtypes = [p, p, p, p, p, p, i64, i64, i64, i32, p, p, p, f32, p, i32, p, i32, i64,
                                               p, ctypes.c_size_t, p, p]
    lib.ue5m3_quantize_fp4_operand_both.restype = i32
    lib.ue5m3_quantize_fp4_operand_both.argtypes = [p, i32, i64, i64, i32, p, f32, i32, p, p, p, p, p, p, p, p, p]
    lib.ue5m3_philox_bytes.restype = i32
    lib.ue5m3_philox_bytes.argtypes = [p, i64, p, p]
    lib.ue5m3_gemm_fp4.restype = i32
    lib.ue5m3_gemm_fp4.argtypes = [p, p, p, p, i64, i64, i64, i32, i32, p, p, p, f32, p, i32, p, i32, i64, p, p, p, p]
    lib.ue5m3_scale_byte_histogram.restype = i32
    lib.ue5m3_scale_byte_histogram.argtypes = [p, i64, i64, i32, i32, p, p]
    lib.ue5m3_place_row_windows.restype = i32
    lib.ue5m3_place_row_windows.argtypes = [p, p, p, i64, i32, p, p, p, i64, i32, i64, p]
    lib.ue5m3_test_e2m1_cvt.restype = i32
    lib.ue5m3_test_e2m1_cvt.argtypes = [ctypes.c_uint32, ctypes.c_uint64, p, p, p]
    if hasattr(lib, "ue5m3_amax_static"):
        lib.ue5m3_amax_static.restype = i32
        lib.ue5m3_amax_static.argtypes = [p, i32, i64, p, p]
    if lib.ue5m3_abi_version() != 2:
        raise NativeLibraryError("ABI version mismatch between the Python package and the library")
    _lib = lib
    return lib


launch_count = 0  # successful kernel-launching library calls of this process


def check(status: int, what: str, launches: int = 1) -> None:
    """Raise on a non-zero status; ``launches`` = kernels the successful call put on the stream."""

    global launch_count
    if status == UE5M3_OK:
        launch_count += launches
        return
    lib = load()
    text = lib.ue5m3_status_string(status).decode()
    if status == 6:
        text += ": " + lib.ue5m3_last_cuda_error().decode()
    raise NativeLibraryError(f"{what} failed: {text} (status {status})")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype is torch.bfloat16:
        return DTYPE_BF16
    if dtype is torch.float32:
        return DTYPE_FP32
    raise TypeError(f"unsupported dtype {dtype}; expected bfloat16 or float32")


def ptr(tensor) -> int | None:
    """Device pointer of a tensor (or of the key tensor of a counter-based bit stream)."""

    if tensor is None:
        return None
    key = getattr(tensor, "key", None)
    return key.data_ptr() if key is not None else tensor.data_ptr()


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_amax_scratch: dict[tuple[int, int], torch.Tensor] = {}


def amax_scratch(device: torch.device) -> torch.Tensor:
    """Zero-initialised reduction scratch, one per (device, stream)."""

    stream = torch.cuda.current_stream(device)
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream.cuda_stream)
    scratch = _amax_scratch.get(key)
    if scratch is None:
        size = load().ue5m3_amax_scratch_bytes()
        scratch = torch.zeros(size, dtype=torch.uint8, device=device)
        _amax_scratch[key] = scratch
    return scratch
