"""ctypes/numpy front end of the C oracle (oracle/ue5m3_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline legs of bench.py.  The shipped package never imports it.

Each function restates the reference behaviour cited in the C source; parity is
pinned by tests/test_oracle_golden.py against the reference's own known-answer
tests and against fixtures generated from the reference's formats.py.
"""

from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

try:  # package import (tests, bench) and script import both work
    from .build import build as _build
except ImportError:  # pragma: no cover
    from build import build as _build

ROUND_TTE = 0
ROUND_SR = 7
BLOCK_ROW = 0
BLOCK_COL = 1
BLOCK_2D = 2

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _build()
        handle = ctypes.CDLL(str(path))
        f32 = ctypes.c_float
        i64 = ctypes.c_int64
        p = ctypes.c_void_p
        handle.ue5m3o_round_magnitude.restype = f32
        handle.ue5m3o_round_magnitude.argtypes = [f32, ctypes.c_int, ctypes.c_int, f32, ctypes.c_int, ctypes.c_int]
        handle.ue5m3o_round_e2m1.restype = f32
        handle.ue5m3o_round_e2m1.argtypes = [f32, ctypes.c_int, ctypes.c_int]
        handle.ue5m3o_round_ue5m3.restype = f32
        handle.ue5m3o_round_ue5m3.argtypes = [f32]
        handle.ue5m3o_e2m1_code.restype = ctypes.c_uint8
        handle.ue5m3o_e2m1_code.argtypes = [f32]
        handle.ue5m3o_e2m1_value.restype = f32
        handle.ue5m3o_e2m1_value.argtypes = [ctypes.c_uint8]
        handle.ue5m3o_ue5m3_code.restype = ctypes.c_uint8
        handle.ue5m3o_ue5m3_code.argtypes = [f32]
        handle.ue5m3o_ue5m3_value.restype = f32
        handle.ue5m3o_ue5m3_value.argtypes = [ctypes.c_uint8]
        handle.ue5m3o_tensor_scales.restype = None
        handle.ue5m3o_tensor_scales.argtypes = [f32, f32, p, p]
        handle.ue5m3o_amax.restype = f32
        handle.ue5m3o_amax.argtypes = [p, i64]
        handle.ue5m3o_quantize.restype = ctypes.c_int
        handle.ue5m3o_quantize.argtypes = [p, i64, i64, ctypes.c_int, ctypes.c_int, f32, f32, ctypes.c_int, p, p, p, p, p, p, p]
        handle.ue5m3o_dequantize.restype = ctypes.c_int
        handle.ue5m3o_dequantize.argtypes = [p, p, i64, i64, ctypes.c_int, ctypes.c_int, f32, f32, p]
        handle.ue5m3o_add_rz.restype = f32
        handle.ue5m3o_add_rz.argtypes = [f32, f32]
        handle.ue5m3o_snap_1024.restype = f32
        handle.ue5m3o_snap_1024.argtypes = [f32]
        handle.ue5m3o_gemm_issue_rz.restype = ctypes.c_int
        handle.ue5m3o_gemm_issue_rz.argtypes = [p, p, i64, i64, i64, ctypes.c_int, p, p, p]
        handle.ue5m3o_gemm_issue_rule.restype = ctypes.c_int
        handle.ue5m3o_gemm_issue_rule.argtypes = [p, p, i64, i64, i64, ctypes.c_int, p, p, p, ctypes.c_int]
        handle.ue5m3o_alpha.restype = f32
        handle.ue5m3o_alpha.argtypes = [f32, f32, f32, f32, ctypes.c_int]
        handle.ue5m3o_rht_b16.restype = ctypes.c_int
        handle.ue5m3o_rht_b16.argtypes = [p, i64, i64, p]
        handle.ue5m3o_num_threads.restype = ctypes.c_int
        handle.ue5m3o_set_threads.restype = None
        handle.ue5m3o_set_threads.argtypes = [ctypes.c_int]
        _lib = handle
    return _lib


def _ptr(array: np.ndarray | None):
    return None if array is None else array.ctypes.data_as(ctypes.c_void_p)


def round_e2m1(values, rounding=ROUND_TTE, rbits=None) -> np.ndarray:
    values = np.asarray(values, dtype=np.float32)
    flat = values.reshape(-1)
    bits = np.zeros(flat.shape, np.int64) if rbits is None else np.asarray(rbits).reshape(-1)
    out = np.array([lib().ue5m3o_round_e2m1(float(v), rounding, int(r)) for v, r in zip(flat, bits)], dtype=np.float32)
    return out.reshape(values.shape)


def round_ue5m3(values) -> np.ndarray:
    values = np.asarray(values, dtype=np.float32)
    out = np.array([lib().ue5m3o_round_ue5m3(float(v)) for v in values.reshape(-1)], dtype=np.float32)
    return out.reshape(values.shape)


def tensor_scales(amax: float, target: float) -> tuple[float, float]:
    enc = ctypes.c_float()
    dec = ctypes.c_float()
    lib().ue5m3o_tensor_scales(amax, target, ctypes.byref(enc), ctypes.byref(dec))
    return enc.value, dec.value


def rht_b16(x: np.ndarray) -> np.ndarray:
    """Fixed-sign normalized B=16 Hadamard transform along the last axis, BF16 result as fp32
    (nn/linear.py:80-114 of the reference)."""

    x = np.ascontiguousarray(x, dtype=np.float32)
    if x.ndim != 2 or x.shape[1] % 16:
        raise ValueError("the B=16 transform expects a rank-2 operand whose last dimension is divisible by 16")
    out = np.empty_like(x)
    if lib().ue5m3o_rht_b16(_ptr(x), x.shape[0], x.shape[1], _ptr(out)):
        raise ValueError("ue5m3o_rht_b16 failed")
    return out


def amax(x: np.ndarray) -> float:
    x = np.ascontiguousarray(x, dtype=np.float32)
    return float(lib().ue5m3o_amax(_ptr(x), x.size))


def scale_grid_shape(rows: int, cols: int, block: int, blocking: int) -> tuple[int, int]:
    br = 1 if blocking == BLOCK_ROW else block
    bc = 1 if blocking == BLOCK_COL else block
    return (rows + br - 1) // br, (cols + bc - 1) // bc


def quantize(
    x: np.ndarray,
    *,
    block: int,
    blocking: int = BLOCK_ROW,
    amax_value: float | None = None,
    target: float = 448.0,
    rounding: int = ROUND_TTE,
    rbits: np.ndarray | None = None,
) -> dict[str, np.ndarray]:
    """Quantize a rank-2 fp32 array; every output is in the orientation of ``x``."""

    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    if amax_value is None:
        amax_value = amax(x)
    grid = scale_grid_shape(rows, cols, block, blocking)
    nibbles = np.empty((rows, cols), np.uint8)
    scale_codes = np.empty(grid, np.uint8)
    block_amax = np.empty(grid, np.float32)
    encoded = np.empty((rows, cols), np.float32)
    dequant = np.empty((rows, cols), np.float32)
    decoded = np.empty((rows, cols), np.float32)
    bits = None
    if rbits is not None:
        bits = np.ascontiguousarray(rbits, dtype=np.uint8)
        assert bits.shape == x.shape
    status = lib().ue5m3o_quantize(
        _ptr(x), rows, cols, block, blocking, amax_value, target, rounding, _ptr(bits),
        _ptr(nibbles), _ptr(scale_codes), _ptr(block_amax), _ptr(encoded), _ptr(dequant), _ptr(decoded),
    )
    if status:
        raise ValueError(f"oracle quantize failed with status {status}")
    return {
        "nibbles": nibbles,
        "scale_codes": scale_codes,
        "block_amax": block_amax,
        "encoded": encoded,
        "dequant": dequant,
        "decoded": decoded,
        "amax": np.float32(amax_value),
    }


def pack_nibbles(nibbles: np.ndarray) -> np.ndarray:
    """Pack [R, C] nibbles into [R, ceil(C/2)] bytes, even element in the low nibble."""

    rows, cols = nibbles.shape
    padded = np.zeros((rows, (cols + 1) // 2 * 2), np.uint8)
    padded[:, :cols] = nibbles
    return (padded[:, 0::2] | (padded[:, 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(packed: np.ndarray, cols: int) -> np.ndarray:
    rows = packed.shape[0]
    out = np.empty((rows, packed.shape[1] * 2), np.uint8)
    out[:, 0::2] = packed & 0xF
    out[:, 1::2] = packed >> 4
    return out[:, :cols]


def scale_values(codes: np.ndarray) -> np.ndarray:
    table = np.array([lib().ue5m3o_ue5m3_value(i) for i in range(256)], dtype=np.float32)
    return table[codes]


def dequantize(nibbles, scale_codes, *, block, blocking, amax_value, target=448.0) -> np.ndarray:
    nibbles = np.ascontiguousarray(nibbles, dtype=np.uint8)
    scale_codes = np.ascontiguousarray(scale_codes, dtype=np.uint8)
    rows, cols = nibbles.shape
    out = np.empty((rows, cols), np.float32)
    lib().ue5m3o_dequantize(_ptr(nibbles), _ptr(scale_codes), rows, cols, block, blocking, amax_value, target, _ptr(out))
    return out


# Alignment window of the FP4 tensor-core accumulation.  Measured on 1.7 million adversarial
# outputs (block scales 2^-6..2^8 on both operands): 35 leaves 7 outputs unexplained, 34 leaves
# 200, 36 leaves 50, no window (exact sum) 47; operands within 30 binades: none, for any value.
NATIVE_WINDOW_BITS = 35


def add_rz(a: float, b: float) -> float:
    return float(lib().ue5m3o_add_rz(a, b))


def snap_1024(c: float) -> float:
    return float(lib().ue5m3o_snap_1024(c))


def alpha(amax_a: float, amax_b: float, target_a: float, target_b: float, reciprocal_form: bool = True) -> float:
    return float(lib().ue5m3o_alpha(amax_a, amax_b, target_a, target_b, int(reciprocal_form)))


def gemm_issue_rz(a: np.ndarray, bt: np.ndarray, *, snap: bool, alpha_value: float | None = None,
                  native_rule: bool = False, native_window: int = NATIVE_WINDOW_BITS) -> np.ndarray:
    """C = A[M,K] @ Bt[N,K]^T under the K=64 issue / RTZ model (fp32 in, fp32 out).

    ``native_rule``: instead of the model's two roundings per issue (partial to nearest, then
    a round-toward-zero add) apply what the FP4 tensor-core instruction was measured to do:
    the four exact 16-block sums of the issue and the accumulator are aligned to the largest
    of them, truncated toward zero ``native_window`` bits below it, added exactly and truncated
    toward zero to fp32 - which is c = RTZ(c + exact issue sum) whenever the addends lie within
    the window."""

    a = np.ascontiguousarray(a, dtype=np.float32)
    bt = np.ascontiguousarray(bt, dtype=np.float32)
    m, k = a.shape
    n, k2 = bt.shape
    assert k == k2
    out = np.empty((m, n), np.float32)
    inexact = ctypes.c_int(0)
    alpha_c = None if alpha_value is None else ctypes.c_float(alpha_value)
    status = lib().ue5m3o_gemm_issue_rule(
        _ptr(a), _ptr(bt), m, n, k, int(snap),
        None if alpha_c is None else ctypes.byref(alpha_c), _ptr(out), ctypes.byref(inexact),
        int(native_window) if native_rule else 0,
    )
    if status:
        raise ValueError(f"oracle gemm failed with status {status}")
    if inexact.value:
        raise ArithmeticError("an issue group spans more binades than the 128-bit oracle accumulator holds")
    return out


def probe_matched_fp4_gemm(
    a: np.ndarray,
    b_t: np.ndarray,
    *,
    block: int,
    target_a: float = 448.0,
    target_b: float = 448.0,
    amax_a: float | None = None,
    amax_b: float | None = None,
    rounding_a: int = ROUND_TTE,
    rounding_b: int = ROUND_TTE,
    rbits_a: np.ndarray | None = None,
    rbits_b_t: np.ndarray | None = None,
    two_dimensional_b: bool = False,
    snap: bool = True,
    reciprocal_alpha: bool = True,
) -> np.ndarray:
    """Full composition of backends/triton/api.py:23-83 on A[M,K] and B^T[N,K].

    B is passed transposed (``b_t[n, k] = B[k, n]``), so its reduction axis is
    the last axis and 1-D blocks of B run along rows of ``b_t`` exactly like A.
    """

    a = np.ascontiguousarray(a, dtype=np.float32)
    b_t = np.ascontiguousarray(b_t, dtype=np.float32)
    if amax_a is None:
        amax_a = amax(a)
    if amax_b is None:
        amax_b = amax(b_t)
    qa = quantize(a, block=block, blocking=BLOCK_ROW, amax_value=amax_a, target=target_a, rounding=rounding_a, rbits=rbits_a)
    qb = quantize(
        b_t, block=block, blocking=BLOCK_2D if two_dimensional_b else BLOCK_ROW,
        amax_value=amax_b, target=target_b, rounding=rounding_b, rbits=rbits_b_t,
    )
    al = alpha(amax_a, amax_b, target_a, target_b, reciprocal_alpha)
    return gemm_issue_rz(qa["encoded"], qb["encoded"], snap=snap, alpha_value=al)


def set_threads(n: int) -> None:
    lib().ue5m3o_set_threads(int(n))


def num_threads() -> int:
    return int(lib().ue5m3o_num_threads())
