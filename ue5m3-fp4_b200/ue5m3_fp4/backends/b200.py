"""Python front end of the sm_100a kernels: tensor amax, packed block quantizer,
packed dequantizer and the probe-matched issue-RZ GEMM.

Every function hands raw device pointers to the C ABI (include/ue5m3_fp4.h) on the
caller's current CUDA stream.  Nothing here computes on the host, and nothing
falls back to another implementation.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import Tensor

from ue5m3_fp4 import _native
from ue5m3_fp4._native import BLOCK_2D, BLOCK_COL, BLOCK_ROW
from ue5m3_fp4.formats import RoundingMode, normalize_rounding

_FAKE_DOMAINS = {
    None: _native.FAKE_NONE,
    "encoded": _native.FAKE_ENCODED,
    "decoded": _native.FAKE_DECODED,
    "dequant": _native.FAKE_DEQUANT,
}


def available() -> bool:
    """True when a CUDA device is visible and the sm_100a library is built."""

    return bool(torch.cuda.is_available() and _native.library_path().exists())


def _require_cuda(tensor: Tensor, name: str) -> None:
    if not isinstance(tensor, Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not tensor.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor; the B200 backend has no CPU path")


def tensor_amax(tensor: Tensor) -> Tensor:
    """max|x| as a 0-dim fp32 device tensor, one HBM pass, no host sync.

    A non-finite input yields +inf or NaN.  Replaces scaling/training.py:39.
    """

    _require_cuda(tensor, "tensor")
    flat = tensor.detach()
    if not flat.is_contiguous():
        flat = flat.contiguous()
    if flat.numel() == 0:
        raise ValueError("cannot take the amax of an empty tensor")
    out = torch.empty((), dtype=torch.float32, device=flat.device)
    scratch = _native.amax_scratch(flat.device)
    with torch.cuda.device(flat.device):
        status = _native.load().ue5m3_amax(
            flat.data_ptr(), _native.dtype_code(flat.dtype), flat.numel(), out.data_ptr(),
            scratch.data_ptr(), scratch.numel(), _native.stream_ptr(flat.device),
        )
    _native.check(status, "ue5m3_amax")
    return out


def global_encode_multiplier(reference: Tensor, scale_target: float) -> Tensor:
    """enc = min(fl(6T)/amax, FLT_MAX), 1 when amax == 0 (formats.py:394-407); metadata only."""

    numerator = torch.tensor(scale_target * 6.0, dtype=torch.float32, device=reference.device)
    raw = numerator / reference
    limit = torch.full_like(raw, torch.finfo(torch.float32).max)
    return torch.where(reference == 0, torch.ones_like(raw), torch.minimum(raw, limit))


_scale_tables: dict[torch.device, Tensor] = {}


def scale_bytes_to_values(scale_bytes: Tensor) -> Tensor:
    """UE5M3 byte (E<<3 | M, bias 15, subnormal M * 2^-17) -> fp32 value; metadata only."""

    table = _scale_tables.get(scale_bytes.device)
    if table is None:
        codes = torch.arange(256, dtype=torch.float64)
        exponent = torch.div(codes, 8, rounding_mode="floor")
        mantissa = codes % 8
        values = torch.where(
            exponent == 0,
            mantissa * 2.0**-17,
            (8 + mantissa) * torch.exp2(exponent - 18),
        )
        table = values.to(torch.float32).to(scale_bytes.device)
        _scale_tables[scale_bytes.device] = table
    return table[scale_bytes.long()]


@dataclass(slots=True)
class PackedOperand:
    """Outputs of one quantizer launch; fields a geometry does not produce are None."""

    rows: int
    cols: int
    block_size: int
    blocking: int
    codes: Tensor | None = None  # [rows, ceil(cols/2)] u8
    scales: Tensor | None = None  # ROW [rows, ceil(cols/B)]; 2D [ceil(rows/B), ceil(cols/B)]
    codes_t: Tensor | None = None  # [cols, ceil(rows/2)] u8
    scales_t: Tensor | None = None  # COL [cols, ceil(rows/B)]; 2D [ceil(cols/B), ceil(rows/B)]
    fake: Tensor | None = None  # [rows, cols]
    fake_t: Tensor | None = None  # [cols, rows]


@dataclass(slots=True)
class PhiloxBits:
    """Random bytes that are never materialised: the kernels compute the byte of element e as
    byte e % 16 of Philox4x32-10(key = seed, counter = {e / 16, stream}).  ``key`` is an int64
    device tensor {seed, stream}.  The reference draws a bit tensor from a torch generator
    (nn/linear.py:371-384); its values are not reproducible by any kernel, so parity for this
    mode is against the explicit bytes returned by ``materialize``."""

    key: Tensor

    @classmethod
    def draw(cls, device: torch.device, generator: torch.Generator | None = None) -> "PhiloxBits":
        key = torch.randint(-(2 ** 62), 2 ** 62, (2,), dtype=torch.int64, device=device, generator=generator)
        return cls(key)

    @property
    def device(self) -> torch.device:
        return self.key.device

    def materialize(self, shape) -> Tensor:
        """The uint8 tensor of this stream for an operand of ``shape`` (row-major elements)."""

        count = 1
        for extent in shape:
            count *= int(extent)
        out = torch.empty(tuple(shape), dtype=torch.uint8, device=self.key.device)
        with torch.cuda.device(self.key.device):
            status = _native.load().ue5m3_philox_bytes(self.key.data_ptr(), count, out.data_ptr(),
                                                       _native.stream_ptr(self.key.device))
        _native.check(status, "ue5m3_philox_bytes")
        return out


def _check_bits(random_bits, x: Tensor) -> None:
    if isinstance(random_bits, PhiloxBits):
        if random_bits.device != x.device or random_bits.key.dtype is not torch.int64 or random_bits.key.numel() != 2:
            raise ValueError("the Philox key must be two int64 values on the operand's device")
        return
    if random_bits.shape != x.shape or random_bits.device != x.device or not random_bits.is_contiguous():
        raise ValueError("random bits must be contiguous, on the operand's device and of its shape")


def _bits_code(bits) -> int:
    if bits is None:
        return _native.BITS_NONE
    if isinstance(bits, PhiloxBits):
        return _native.BITS_PHILOX
    if bits.dtype is torch.uint8:
        return _native.BITS_U8
    if bits.dtype is torch.int32:
        return _native.BITS_I32
    raise TypeError("random bits must have dtype int32 or uint8")


def quantize_packed(
    x: Tensor,
    *,
    block_size: int,
    blocking: int = BLOCK_ROW,
    tensor_amax: Tensor,
    scale_target: float = 448.0,
    rounding: str | RoundingMode = RoundingMode.TIES_TO_EVEN,
    random_bits: Tensor | None = None,
    packed: bool = True,
    packed_t: bool | None = None,
    fake_domain: str | None = None,
    fake_dtype: torch.dtype | None = None,
    fake: bool | None = None,
    fake_t: bool = False,
) -> PackedOperand:
    """One fused quantizer launch on a rank-2 contiguous bf16/fp32 CUDA tensor.

    ``tensor_amax`` is a one-element fp32 device tensor (the held reference); it is
    read on the device.  ``packed`` / ``packed_t`` select the natural / transposed
    packed outputs (transposed = reduction axis contiguous for COL and 2D blocks),
    ``fake`` / ``fake_t`` the value tensors of ``fake_domain``.
    """

    _require_cuda(x, "x")
    if x.ndim != 2 or not x.is_contiguous():
        raise ValueError("x must be a contiguous rank-2 tensor")
    if tensor_amax.device != x.device or tensor_amax.dtype is not torch.float32 or tensor_amax.numel() != 1:
        raise ValueError("tensor_amax must be a one-element float32 tensor on the operand's device")
    if block_size not in (16, 32):
        raise ValueError("block_size must be 16 or 32")
    mode = normalize_rounding(rounding)
    stochastic = mode is RoundingMode.STOCHASTIC_8BIT_MIDPOINT
    if stochastic:
        if random_bits is None:
            raise ValueError("stochastic rounding requires explicit random bits")
        _check_bits(random_bits, x)
    elif random_bits is not None:
        raise ValueError("random bits are only valid with stochastic rounding")
    rows, cols = x.shape
    dev = x.device
    domain = _FAKE_DOMAINS[fake_domain]
    if fake is None:
        fake = fake_domain is not None and not fake_t
    if (fake or fake_t) and domain == _native.FAKE_NONE:
        raise ValueError("fake outputs need a fake_domain")
    if fake_dtype is None:
        fake_dtype = x.dtype
    if packed_t is None:
        packed_t = blocking != BLOCK_ROW and packed
    nb_r, nb_c = (rows + block_size - 1) // block_size, (cols + block_size - 1) // block_size
    result = PackedOperand(rows, cols, block_size, blocking)
    u8 = torch.uint8
    if blocking == BLOCK_ROW:
        if packed_t or fake_t:
            raise ValueError("row blocks have no transposed outputs")
        if packed:
            result.codes = torch.empty((rows, (cols + 1) // 2), dtype=u8, device=dev)
            result.scales = torch.empty((rows, nb_c), dtype=u8, device=dev)
    elif blocking == BLOCK_COL:
        if packed_t:
            result.codes_t = torch.empty((cols, (rows + 1) // 2), dtype=u8, device=dev)
            result.scales_t = torch.empty((cols, nb_r), dtype=u8, device=dev)
    elif blocking == BLOCK_2D:
        if packed:
            result.codes = torch.empty((rows, (cols + 1) // 2), dtype=u8, device=dev)
            result.scales = torch.empty((nb_r, nb_c), dtype=u8, device=dev)
        if packed_t:
            result.codes_t = torch.empty((cols, (rows + 1) // 2), dtype=u8, device=dev)
            result.scales_t = torch.empty((nb_c, nb_r), dtype=u8, device=dev)
    else:
        raise ValueError("unknown block geometry")
    if fake:
        result.fake = torch.empty((rows, cols), dtype=fake_dtype, device=dev)
    if fake_t:
        result.fake_t = torch.empty((cols, rows), dtype=fake_dtype, device=dev)
    with torch.cuda.device(dev):
        status = _native.load().ue5m3_quantize(
            x.data_ptr(), _native.dtype_code(x.dtype), rows, cols, block_size, blocking,
            tensor_amax.data_ptr(), float(scale_target),
            _native.ROUND_STOCHASTIC_FAST if stochastic else _native.ROUND_TIES_TO_EVEN,
            _native.ptr(random_bits), _bits_code(random_bits),
            _native.ptr(result.codes), _native.ptr(result.scales),
            _native.ptr(result.codes_t), _native.ptr(result.scales_t),
            _native.ptr(result.fake), _native.ptr(result.fake_t),
            _native.dtype_code(fake_dtype), domain, _native.stream_ptr(dev),
        )
    _native.check(status, "ue5m3_quantize")
    return result


def dequantize_packed(
    codes: Tensor,
    scales: Tensor,
    *,
    rows: int,
    cols: int,
    block_size: int,
    two_dimensional: bool,
    tensor_amax: Tensor,
    scale_target: float = 448.0,
    out_dtype: torch.dtype = torch.float32,
) -> Tensor:
    """Packed nibbles + scale bytes -> p * (s * dec)  (formats.py:439,450)."""

    _require_cuda(codes, "codes")
    out = torch.empty((rows, cols), dtype=out_dtype, device=codes.device)
    with torch.cuda.device(codes.device):
        status = _native.load().ue5m3_dequantize(
            codes.data_ptr(), scales.data_ptr(), rows, cols, block_size, int(two_dimensional),
            tensor_amax.data_ptr(), float(scale_target), out.data_ptr(), _native.dtype_code(out_dtype),
            _native.stream_ptr(codes.device),
        )
    _native.check(status, "ue5m3_dequantize")
    return out


@dataclass(slots=True)
class EpilogueAlpha:
    """alpha of a GEMM epilogue given by its ingredients: the two held tensor amaxes (device
    scalars) and the fp32 reciprocal of (Ta*6)*(Tb*6).  The kernels form
    fl(fl(amax_a*amax_b) * inv_denominator) themselves, which is the value
    ``encoded_global_alpha`` computes with two ATen launches."""

    amax_a: Tensor
    amax_b: Tensor
    inv_denominator: float

    @classmethod
    def of(cls, amax_a: Tensor, amax_b: Tensor, target_a: float, target_b: float) -> "EpilogueAlpha":
        import numpy as np

        denominator = np.float32((float(target_a) * 6.0) * (float(target_b) * 6.0))
        return cls(amax_a.reshape(1), amax_b.reshape(1), float(np.float32(1.0) / denominator))


def _alpha_arguments(alpha, device: torch.device) -> tuple:
    """(alpha_dev, amax_a_dev, amax_b_dev, inv_denominator) of the C ABI."""

    if alpha is None:
        return (None, None, None, 0.0)
    if isinstance(alpha, EpilogueAlpha):
        for value in (alpha.amax_a, alpha.amax_b):
            if value.dtype is not torch.float32 or value.numel() != 1 or value.device != device:
                raise ValueError("tensor amaxes must be one-element float32 tensors on the operands' device")
        return (None, alpha.amax_a.data_ptr(), alpha.amax_b.data_ptr(), alpha.inv_denominator)
    if alpha.dtype is not torch.float32 or alpha.numel() != 1 or alpha.device != device:
        raise ValueError("alpha must be a one-element float32 tensor on the operands' device")
    return (alpha.data_ptr(), None, None, 0.0)


_status_words: dict[torch.device, Tensor] = {}


def gemm_status(device: torch.device) -> Tensor:
    """Device int32[4] written by the GEMM when a bounded wait expires (all zero = healthy)."""

    words = _status_words.get(device)
    if words is None:
        words = torch.zeros(4, dtype=torch.int32, device=device)
        _status_words[device] = words
    return words


def _raise_on_status(words, device: torch.device) -> None:
    if words[0]:
        gemm_status(device).zero_()
        raise RuntimeError(
            f"GEMM kernel gave up on a bounded wait (site {words[1]}, issue {words[2]}, tile {words[3]}); "
            "the outputs of that launch and of every GEMM launched after it are invalid"
        )


def check_gemm_status(device: torch.device) -> None:
    """Synchronising check of the GEMM status words; raises if a wait expired."""

    _raise_on_status(gemm_status(device).tolist(), device)


_status_polls: dict[torch.device, tuple[Tensor, torch.cuda.Event]] = {}


def poll_gemm_status(device: torch.device) -> None:
    """Check of the GEMM status words that never blocks the host: looks at the copy requested by
    the previous call (if it has arrived) and requests the next one.  ``TrainingScaleState.begin_step``
    and the inference controller call it once per step / phase change, so a kernel that gave up on
    a bounded wait stops the run within two steps instead of feeding unwritten outputs onward."""

    pending = _status_polls.get(device)
    if pending is not None:
        host, event = pending
        if not event.query():
            return
        _raise_on_status(host.tolist(), device)
    else:
        host = torch.empty(4, dtype=torch.int32, pin_memory=True)
        event = torch.cuda.Event()
    host.copy_(gemm_status(device), non_blocking=True)
    event.record(torch.cuda.current_stream(device))
    _status_polls[device] = (host, event)


def gemm_issue_rz(
    a: Tensor,
    bt: Tensor,
    *,
    snap: bool,
    alpha: "Tensor | EpilogueAlpha | None" = None,
    bias: Tensor | None = None,
    out_dtype: torch.dtype = torch.float32,
) -> Tensor:
    """out[M,N] = epilogue(A[M,K] @ Bt[N,K]^T) on bf16 K-major operands (issue-RZ model)."""

    _require_cuda(a, "a")
    _require_cuda(bt, "bt")
    if a.dtype is not torch.bfloat16 or bt.dtype is not torch.bfloat16:
        raise TypeError("a and b must have dtype bfloat16")
    if a.ndim != 2 or bt.ndim != 2 or a.shape[1] != bt.shape[1]:
        raise ValueError("a and b have incompatible K dimensions")
    if not a.is_contiguous() or not bt.is_contiguous():
        raise ValueError("a and b must be contiguous")
    m, k = a.shape
    n = bt.shape[0]
    if k % 64:
        raise ValueError("K must be divisible by 64")
    out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    if m == 0 or n == 0:
        return out
    alpha_args = _alpha_arguments(alpha, a.device)
    if bias is not None:
        if bias.numel() != n or bias.device != a.device or not bias.is_contiguous():
            raise ValueError("bias must be a contiguous vector of length N on the operands' device")
    with torch.cuda.device(a.device):
        status = _native.load().ue5m3_gemm_issue_rz_bf16(
            a.data_ptr(), bt.data_ptr(), m, n, k, int(bool(snap)), *alpha_args,
            _native.ptr(bias), _native.dtype_code(bias.dtype) if bias is not None else 0,
            out.data_ptr(), _native.dtype_code(out_dtype), n, gemm_status(a.device).data_ptr(),
            _native.stream_ptr(a.device),
        )
    _native.check(status, "ue5m3_gemm_issue_rz_bf16")
    return out


FALLBACK_MAX_ROWS = 4096  # UE5M3_FALLBACK_MAX_ROWS of the C ABI


def new_window_record(rows: int, device: torch.device) -> Tensor:
    """Zeroed window record of an operand with ``rows`` rows (layout: include/ue5m3_fp4.h): the
    quantizer lists here the rows that hold a block scale outside the tensor core's UE4M3 range."""

    count = _native.load().ue5m3_window_record_ints(rows)
    padded = (count + 3) & ~3   # slices stay 16-byte aligned
    if padded > _RECORD_CHUNK_INTS // 4:
        return torch.zeros(count, dtype=torch.int32, device=device)
    # Records are small and needed by the dozen per layer step: they are cut from a zeroed chunk
    # (one fill launch per chunk instead of one per record).  A chunk belongs to one stream, so
    # its fill is ordered before every kernel that uses a slice; an exhausted chunk lives on for
    # as long as any of its slices does.
    key = (device, _native.stream_ptr(device) or 0)
    chunk, used = _record_chunks.get(key, (None, 0))
    if chunk is None or used + padded > chunk.numel():
        chunk, used = torch.zeros(_RECORD_CHUNK_INTS, dtype=torch.int32, device=device), 0
    _record_chunks[key] = (chunk, used + padded)
    return chunk[used:used + count]


_RECORD_CHUNK_INTS = 1 << 22   # 16 MiB
_record_chunks: dict[tuple[torch.device, int], tuple[Tensor, int]] = {}


def scale_shift_for_target(scale_target: float) -> int:
    """Power-of-two re-bias of a tensor's block scales: scales up to the target (with the
    ties-to-even slack of one sixteenth) must not exceed UE4M3's maximum 448."""

    return max(0, math.ceil(math.log2(scale_target / 448.0)))


def pack_scales(scales: Tensor, *, rows: int, k: int, block_size: int, two_dimensional: bool, shift: int,
                record: Tensor | None = None, want_raw: bool = False):
    """UE5M3 scale bytes of a K-major operand -> UE4M3 bytes in the tensor core's scale layout
    (and, with ``want_raw``, the unmodified bytes in the same layout).  ``record``: the operand's
    window record; a fresh one is made when it is not given."""

    _require_cuda(scales, "scales")
    size = _native.load().ue5m3_packed_scales_bytes(rows, k)
    if size == 0:
        raise ValueError("K must be divisible by 64")
    out = torch.empty(size, dtype=torch.uint8, device=scales.device)
    raw = torch.empty(size, dtype=torch.uint8, device=scales.device) if want_raw else None
    if record is None:
        record = new_window_record(rows, scales.device)
    with torch.cuda.device(scales.device):
        status = _native.load().ue5m3_pack_scales_ue4m3(
            scales.data_ptr(), rows, k, block_size, int(two_dimensional), shift, out.data_ptr(),
            _native.ptr(raw), record.data_ptr(), _native.stream_ptr(scales.device),
        )
    _native.check(status, "ue5m3_pack_scales_ue4m3")
    return (out, raw, record) if want_raw else out


def gemm_fp4(
    a_codes: Tensor, a_sf: Tensor, b_codes: Tensor, b_sf: Tensor, *, m: int, n: int, k: int, shift_sum: int,
    snap: bool, alpha: "Tensor | EpilogueAlpha | None" = None, bias: Tensor | None = None,
    out_dtype: torch.dtype = torch.float32, a_record: Tensor | None = None, b_record: Tensor | None = None,
) -> Tensor:
    """out[M,N] on packed E2M1 codes + packed scales with the FP4 block-scaled tensor cores;
    ``a_record`` / ``b_record``: window records whose placed rows carry a shift of their own."""

    _require_cuda(a_codes, "a_codes")
    if k % 64:
        raise ValueError("K must be divisible by 64")
    if a_codes.shape != (m, k // 2) or b_codes.shape != (n, k // 2):
        raise ValueError("packed codes must be [rows, K/2] with the reduction axis contiguous")
    out = torch.empty((m, n), dtype=out_dtype, device=a_codes.device)
    with torch.cuda.device(a_codes.device):
        status = _native.load().ue5m3_gemm_fp4(
            a_codes.data_ptr(), a_sf.data_ptr(), b_codes.data_ptr(), b_sf.data_ptr(), m, n, k, shift_sum,
            int(bool(snap)), *_alpha_arguments(alpha, a_codes.device), _native.ptr(bias),
            _native.dtype_code(bias.dtype) if bias is not None else 0, out.data_ptr(),
            _native.dtype_code(out_dtype), n, _native.ptr(a_record), _native.ptr(b_record),
            gemm_status(a_codes.device).data_ptr(), _native.stream_ptr(a_codes.device),
        )
    _native.check(status, "ue5m3_gemm_fp4")
    return out


def gemm_path() -> str:
    """"fp4" (block-scaled FP4 tensor cores, default) or "bf16" (issue-RZ kernel on encoded
    bf16 operands), from the environment variable UE5M3_GEMM_PATH."""

    import os

    path = os.environ.get("UE5M3_GEMM_PATH", "fp4").strip().lower()
    if path not in {"fp4", "bf16"}:
        raise ValueError("UE5M3_GEMM_PATH must be 'fp4' or 'bf16'")
    return path


@dataclass(slots=True)
class Fp4Operand:
    """A K-major packed GEMM operand: codes [rows, K/2], block scales in the tensor-core layout
    (UE4M3, re-biased by ``shift``), the same scales as unmodified UE5M3 bytes, and the window
    record that lists the rows where the two differ (a scale outside the UE4M3 window)."""

    codes: Tensor
    scale_factors: Tensor
    shift: int
    rows: int
    k: int
    raw_scale_factors: Tensor | None = None
    record: Tensor | None = None
    placed: bool = False   # place_row_windows has run on this operand

    def window_counts(self) -> tuple[int, int]:
        """(rows the quantizer flagged, 16-element units outside the window at the tensor's
        shift); synchronises."""

        if self.record is None:
            return (0, 0)
        flagged, units = self.record[:2].tolist()
        return int(flagged), int(units)

    def flagged_rows(self) -> list[int]:
        """Rows with a block scale outside the window at the tensor's shift; synchronises."""

        if self.record is None:
            return []
        flags = self.record[4 + FALLBACK_MAX_ROWS:4 + FALLBACK_MAX_ROWS + self.rows]
        return torch.nonzero(flags).flatten().tolist()

    def placement(self) -> tuple[list[int], dict[int, int]]:
        """After ``place_row_windows``: (rows listed for recomputation, {row: its shift minus the
        tensor's} for rows that got a window of their own); synchronises."""

        if self.record is None:
            return [], {}
        head = self.record[:4].tolist()
        listed = sorted(self.record[4:4 + min(head[2], FALLBACK_MAX_ROWS)].tolist())
        shifts = self.record[4 + FALLBACK_MAX_ROWS + self.rows:4 + FALLBACK_MAX_ROWS + 2 * self.rows]
        placed = {int(r): int(shifts[r]) for r in self.flagged_rows() if r not in set(listed)} if head[3] else {}
        return listed, placed


def quantize_fp4_operand(
    x: Tensor,
    *,
    block_size: int,
    blocking: int,
    transposed: bool,
    tensor_amax: Tensor,
    scale_target: float,
    rounding: str | RoundingMode = RoundingMode.TIES_TO_EVEN,
    random_bits: Tensor | None = None,
    shift_headroom: int = 0,
    hadamard: bool = False,
) -> Fp4Operand:
    """Quantize ``x`` [R, C] into a packed K-major operand of the FP4 GEMM: reduction over C
    (``transposed=False``: ROW or 2-D blocks) or over R (``transposed=True``: COL or 2-D
    blocks, outputs written transposed)."""

    shift = scale_shift_for_target(scale_target) + shift_headroom
    if hadamard:
        if not transposed or blocking != BLOCK_COL or block_size != 16:
            raise ValueError("the fixed-sign B=16 Hadamard transform applies to transposed 16 x 1 operands only")
        return _quantize_fp4_operand_fused(x, block_size, blocking, tensor_amax, scale_target, rounding,
                                           random_bits, shift, transposed=True, hadamard=True)
    if not transposed and blocking in (BLOCK_ROW, BLOCK_2D) and x.ndim == 2 and x.shape[1] % 64 == 0 \
            and x.is_contiguous() and x.data_ptr() % 32 == 0:
        return _quantize_fp4_operand_fused(x, block_size, blocking, tensor_amax, scale_target, rounding,
                                           random_bits, shift)
    if transposed and blocking in (BLOCK_COL, BLOCK_2D) and x.ndim == 2 and x.shape[0] % 64 == 0 \
            and x.is_contiguous():
        return _quantize_fp4_operand_fused(x, block_size, blocking, tensor_amax, scale_target, rounding,
                                           random_bits, shift, transposed=True)
    packed = quantize_packed(
        x, block_size=block_size, blocking=blocking, tensor_amax=tensor_amax, scale_target=scale_target,
        rounding=rounding, random_bits=random_bits, packed=not transposed, packed_t=transposed,
    )
    rows, k = (x.shape[1], x.shape[0]) if transposed else (x.shape[0], x.shape[1])
    codes = packed.codes_t if transposed else packed.codes
    scales = packed.scales_t if transposed else packed.scales
    sf, raw, record = pack_scales(scales, rows=rows, k=k, block_size=block_size,
                                  two_dimensional=blocking == BLOCK_2D, shift=shift, want_raw=True)
    return Fp4Operand(codes, sf, shift, rows, k, raw, record)


def quantize_fp4_operand_both(x: Tensor, *, block_size: int, tensor_amax: Tensor, scale_target: float,
                              shift_headroom: int = 0) -> "tuple[Fp4Operand, Fp4Operand] | None":
    """A weight ``x`` [R, C] with B x B blocks, ties-to-even, as BOTH packed GEMM operands from
    one read: (operand of x, reduction over C; operand of x^T, reduction over R) - bit for bit
    what two ``quantize_fp4_operand`` calls give (ue5m3_quantize_fp4_operand_both).  Returns None
    when the shape does not qualify (both dimensions multiples of 64, contiguous, aligned); the
    caller then makes the two operands separately."""

    _require_cuda(x, "x")
    if x.ndim != 2 or x.shape[0] % 64 or x.shape[1] % 64 or not x.is_contiguous() or x.data_ptr() % 16:
        return None
    if x.dtype not in (torch.bfloat16, torch.float32):
        return None
    if tensor_amax.device != x.device or tensor_amax.dtype is not torch.float32 or tensor_amax.numel() != 1:
        raise ValueError("tensor_amax must be a one-element float32 tensor on the operand's device")
    if block_size not in (16, 32):
        raise ValueError("block_size must be 16 or 32")
    shift = scale_shift_for_target(scale_target) + shift_headroom
    rows, cols = x.shape
    dev = x.device
    lib = _native.load()
    codes = torch.empty((rows, cols // 2), dtype=torch.uint8, device=dev)
    codes_t = torch.empty((cols, rows // 2), dtype=torch.uint8, device=dev)
    sf = torch.empty(lib.ue5m3_packed_scales_bytes(rows, cols), dtype=torch.uint8, device=dev)
    sf_t = torch.empty(lib.ue5m3_packed_scales_bytes(cols, rows), dtype=torch.uint8, device=dev)
    raw, raw_t = torch.empty_like(sf), torch.empty_like(sf_t)
    record, record_t = new_window_record(rows, dev), new_window_record(cols, dev)
    with torch.cuda.device(dev):
        status = lib.ue5m3_quantize_fp4_operand_both(
            x.data_ptr(), _native.dtype_code(x.dtype), rows, cols, block_size, tensor_amax.data_ptr(),
            float(scale_target), shift, codes.data_ptr(), sf.data_ptr(), raw.data_ptr(), record.data_ptr(),
            codes_t.data_ptr(), sf_t.data_ptr(), raw_t.data_ptr(), record_t.data_ptr(), _native.stream_ptr(dev))
    _native.check(status, "ue5m3_quantize_fp4_operand_both")
    return (Fp4Operand(codes, sf, shift, rows, cols, raw, record),
            Fp4Operand(codes_t, sf_t, shift, cols, rows, raw_t, record_t))


def _quantize_fp4_operand_fused(x: Tensor, block_size: int, blocking: int, tensor_amax: Tensor,
                                scale_target: float, rounding, random_bits: Tensor | None, shift: int,
                                *, want_scales: bool = False, transposed: bool = False, hadamard: bool = False):
    """One launch: codes and tensor-core scale atoms (ue5m3_quantize_fp4_operand, or
    ue5m3_quantize_fp4_operand_t for the operand x^T)."""

    _require_cuda(x, "x")
    if tensor_amax.device != x.device or tensor_amax.dtype is not torch.float32 or tensor_amax.numel() != 1:
        raise ValueError("tensor_amax must be a one-element float32 tensor on the operand's device")
    if block_size not in (16, 32):
        raise ValueError("block_size must be 16 or 32")
    mode = normalize_rounding(rounding)
    stochastic = mode is RoundingMode.STOCHASTIC_8BIT_MIDPOINT
    if stochastic:
        if random_bits is None:
            raise ValueError("stochastic rounding requires explicit random bits")
        _check_bits(random_bits, x)
    elif random_bits is not None:
        raise ValueError("random bits are only valid with stochastic rounding")
    dev = x.device
    lib = _native.load()
    if transposed:
        k, rows = x.shape
        codes = torch.empty((rows, k // 2), dtype=torch.uint8, device=dev)
        sf = torch.empty(lib.ue5m3_packed_scales_bytes(rows, k), dtype=torch.uint8, device=dev)
        raw = torch.empty_like(sf)
        record = new_window_record(rows, dev)
        if hadamard:
            if not x.is_contiguous() or k % 64:
                raise ValueError("the transformed operand needs a contiguous tensor whose first dimension is a multiple of 64")
            with torch.cuda.device(dev):
                status = lib.ue5m3_quantize_fp4_operand_t_rht(
                    x.data_ptr(), _native.dtype_code(x.dtype), k, rows, tensor_amax.data_ptr(), float(scale_target),
                    _native.ROUND_STOCHASTIC_FAST if stochastic else _native.ROUND_TIES_TO_EVEN,
                    _native.ptr(random_bits), _bits_code(random_bits), shift,
                    codes.data_ptr(), sf.data_ptr(), raw.data_ptr(), record.data_ptr(), _native.stream_ptr(dev),
                )
            _native.check(status, "ue5m3_quantize_fp4_operand_t_rht")
            return Fp4Operand(codes, sf, shift, rows, k, raw, record)
        with torch.cuda.device(dev):
            status = lib.ue5m3_quantize_fp4_operand_t(
                x.data_ptr(), _native.dtype_code(x.dtype), k, rows, block_size, blocking,
                tensor_amax.data_ptr(), float(scale_target),
                _native.ROUND_STOCHASTIC_FAST if stochastic else _native.ROUND_TIES_TO_EVEN,
                _native.ptr(random_bits), _bits_code(random_bits), shift,
                codes.data_ptr(), sf.data_ptr(), raw.data_ptr(), record.data_ptr(), _native.stream_ptr(dev),
            )
        _native.check(status, "ue5m3_quantize_fp4_operand_t")
        return Fp4Operand(codes, sf, shift, rows, k, raw, record)
    rows, k = x.shape
    codes = torch.empty((rows, k // 2), dtype=torch.uint8, device=dev)
    sf = torch.empty(lib.ue5m3_packed_scales_bytes(rows, k), dtype=torch.uint8, device=dev)
    raw = torch.empty_like(sf)
    record = new_window_record(rows, dev)
    scales = None
    if want_scales:
        scale_rows = rows if blocking == BLOCK_ROW else (rows + block_size - 1) // block_size
        scales = torch.empty((scale_rows, k // block_size), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        status = lib.ue5m3_quantize_fp4_operand(
            x.data_ptr(), _native.dtype_code(x.dtype), rows, k, block_size, blocking,
            tensor_amax.data_ptr(), float(scale_target),
            _native.ROUND_STOCHASTIC_FAST if stochastic else _native.ROUND_TIES_TO_EVEN,
            _native.ptr(random_bits), _bits_code(random_bits), shift,
            codes.data_ptr(), sf.data_ptr(), raw.data_ptr(), _native.ptr(scales),
            record.data_ptr(), _native.stream_ptr(dev),
        )
    _native.check(status, "ue5m3_quantize_fp4_operand")
    operand = Fp4Operand(codes, sf, shift, rows, k, raw, record)
    return (operand, scales) if want_scales else operand


def hadamard_amax_transposed(x: Tensor) -> Tensor:
    """max |y| (one-element fp32 device tensor) of the operand x^T after the TE-settings
    comparator's fixed-sign B=16 Hadamard transform along its reduction axis (the rows of x);
    nn/linear.py:80-114,389-400 of the reference (``_finite_amax`` of the transformed tensor)."""

    _require_cuda(x, "x")
    if x.ndim != 2 or not x.is_contiguous() or x.shape[0] % 16:
        raise ValueError("the reported B=16 RHT requires a contiguous rank-2 operand with the reduced dimension divisible by 16")
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        status = _native.load().ue5m3_rht_amax_t(x.data_ptr(), _native.dtype_code(x.dtype), x.shape[0], x.shape[1],
                                                 out.data_ptr(), _native.stream_ptr(x.device))
    _native.check(status, "ue5m3_rht_amax_t")
    return out


def place_row_windows(a: Fp4Operand | None, b: Fp4Operand | None) -> None:
    """Give the flagged rows of the two operands of one product scale windows of their own where
    their scales fit one, and list the rest for the recomputation pass (ue5m3_place_row_windows;
    one launch, returns at once on the device when nothing is flagged).  Idempotence is not
    needed: ``gemm_fp4_operands`` calls it once per operand pair; an operand that is reused
    (a cached weight) is placed once, the flag of that is kept on the operand."""

    todo = [op for op in (a, b) if op is not None and not op.placed]
    if not todo:
        return
    first = todo[0]
    second = todo[1] if len(todo) > 1 else None
    if second is not None and second.k != first.k:
        raise ValueError("operands of one product share the reduction length")
    for op in todo:
        if op.record is None or op.raw_scale_factors is None:
            raise ValueError("packed operands must carry their raw scales and window records")
    with torch.cuda.device(first.codes.device):
        status = _native.load().ue5m3_place_row_windows(
            first.scale_factors.data_ptr(), first.raw_scale_factors.data_ptr(), first.record.data_ptr(), first.rows,
            first.shift,
            _native.ptr(None if second is None else second.scale_factors),
            _native.ptr(None if second is None else second.raw_scale_factors),
            _native.ptr(None if second is None else second.record), 0 if second is None else second.rows,
            0 if second is None else second.shift, first.k, _native.stream_ptr(first.codes.device),
        )
    _native.check(status, "ue5m3_place_row_windows")
    for op in todo:
        op.placed = True


def scale_byte_histogram(operand: Fp4Operand, *, block_size: int, two_dimensional: bool = False,
                         out: Tensor | None = None) -> Tensor:
    """256 int64 counters: how many blocks of the operand carry each UE5M3 scale byte (bin 0: blocks
    whose elements are all zero; byte 0xF7: saturated).  Accumulates into ``out`` when given.  Reads
    only the operand's raw scale atoms.  The device-side form of the block-scale diagnostics of
    reproduce/scale_target/capture_scale_target_histograms.py:257-366 of the reference."""

    if operand.raw_scale_factors is None:
        raise ValueError("the operand carries no raw scale atoms")
    device = operand.codes.device
    if out is None:
        out = torch.zeros(256, dtype=torch.int64, device=device)
    elif out.dtype is not torch.int64 or out.numel() != 256 or out.device != device or not out.is_contiguous():
        raise ValueError("out must be a contiguous int64 tensor of 256 counters on the operand's device")
    with torch.cuda.device(device):
        status = _native.load().ue5m3_scale_byte_histogram(
            operand.raw_scale_factors.data_ptr(), operand.rows, operand.k, block_size, int(two_dimensional),
            out.data_ptr(), _native.stream_ptr(device))
    _native.check(status, "ue5m3_scale_byte_histogram")
    return out


_window_log: list | None = None


def log_window_records(enable: bool) -> None:
    """Start (or stop and discard) keeping the window records of every FP4 product, for
    ``window_log_summary``; diagnostic, off by default."""

    global _window_log
    _window_log = [] if enable else None


def window_log_summary() -> dict:
    """How many of the logged products had operand rows outside the scale window, and how the
    recomputation pass ran for them; synchronises (one read for all records)."""

    entries = _window_log or []
    if not entries:
        return {"products": 0}
    heads = torch.stack([torch.stack((a[2:4], b[2:4])) for a, b, _ in entries]).tolist()
    summary = {"products": len(entries), "with_listed_rows": 0, "with_listed_columns": 0, "recomputed_in_full": 0,
               "listed_rows_total": 0, "listed_columns_total": 0, "recomputed_tflop": 0.0, "total_tflop": 0.0,
               "in_full_by_shape": {}, "listed_by_shape": {}, "rows_placed_total": 0, "columns_placed_total": 0}
    for ((rows_a, placed_a), (rows_b, placed_b)), (_, _, (m, n, k)) in zip(heads, entries):
        summary["rows_placed_total"] += placed_a
        summary["columns_placed_total"] += placed_b
        flop = 2.0 * m * n * k / 1e12
        summary["total_tflop"] += flop
        shape = f"{m}x{n}x{k}"
        if rows_a > FALLBACK_MAX_ROWS or rows_b > FALLBACK_MAX_ROWS:
            summary["recomputed_in_full"] += 1
            summary["recomputed_tflop"] += flop
            key = f"{shape}:{'A' if rows_a > FALLBACK_MAX_ROWS else ''}{'B' if rows_b > FALLBACK_MAX_ROWS else ''}"
            summary["in_full_by_shape"][key] = summary["in_full_by_shape"].get(key, 0) + 1
            continue
        if rows_a or rows_b:
            summary["listed_by_shape"][shape] = summary["listed_by_shape"].get(shape, 0) + 1
        summary["with_listed_rows"] += rows_a > 0
        summary["with_listed_columns"] += rows_b > 0
        summary["listed_rows_total"] += rows_a
        summary["listed_columns_total"] += rows_b
        summary["recomputed_tflop"] += flop * min(1.0, rows_a / m + rows_b / n)
    return summary


def fallback_mode() -> str:
    """"workspace" (default): the recomputation pass decodes every needed operand row once into a
    per-stream device workspace and runs the TMA-fed issue-RZ kernel on it; "inline"
    (UE5M3_FALLBACK=inline): it decodes per tile inside its own GEMM kernel and needs no memory."""

    import os

    mode = os.environ.get("UE5M3_FALLBACK", "workspace").strip().lower()
    if mode not in ("workspace", "inline"):
        raise ValueError("UE5M3_FALLBACK must be 'workspace' or 'inline'")
    return mode


_fallback_workspaces: dict[tuple[torch.device, int], Tensor] = {}


def _fallback_workspace(device: torch.device, size: int) -> Tensor:
    """Grow-only scratch of the recomputation pass, one per (device, stream): calls on one stream
    are ordered, so consecutive products share it."""

    key = (device, _native.stream_ptr(device) or 0)
    held = _fallback_workspaces.get(key)
    if held is None or held.numel() < size:
        held = torch.empty(size, dtype=torch.uint8, device=device)
        _fallback_workspaces[key] = held
    return held


def fallback_workspace_bytes(m: int, n: int, k: int) -> int:
    """Bytes of workspace that the recomputation pass wants for an [m, k] x [n, k] product:
    (2 x 4096 + m + n) rows of k bf16 values (host arithmetic of ue5m3_fallback_workspace_bytes)."""

    if m <= 0 or n <= 0 or k <= 0:
        return 0
    return (2 * FALLBACK_MAX_ROWS + m + n) * k * 2


def reserve_fallback_workspace(device: torch.device, size: int) -> int:
    """Make the recomputation pass's workspace of ``device``'s current stream at least ``size``
    bytes now; returns the bytes held."""

    with torch.cuda.device(device):
        return _fallback_workspace(torch.device(device), int(size)).numel()


def gemm_fp4_operands(a: Fp4Operand, b: Fp4Operand, *, snap: bool, alpha: "Tensor | EpilogueAlpha | None" = None,
                      bias: Tensor | None = None, out_dtype: torch.dtype = torch.float32,
                      kernel_events: "tuple[torch.cuda.Event, torch.cuda.Event] | None" = None) -> Tensor:
    """FP4 tensor-core product of two packed operands, followed (stream-ordered, no host
    synchronisation) by the recomputation of whatever their window records list: output rows
    for A, output columns for B, everything when a list overflowed.  The recomputation runs the
    issue-RZ BF16 instruction sequence on the exact encoded operands, so the result is the
    reference model's for every UE5M3 scale (the reference has no scale window,
    formats.py:125-134).  ``kernel_events``: a (start, stop) pair recorded directly around the FP4
    GEMM launch itself, for measurements of that kernel alone."""

    if a.k != b.k:
        raise ValueError("a and b have incompatible K dimensions")
    if a.record is None or b.record is None or a.raw_scale_factors is None or b.raw_scale_factors is None:
        raise ValueError("packed operands must carry their raw scales and window records")
    place_row_windows(a, b)
    if kernel_events is not None:
        kernel_events[0].record()
    out = gemm_fp4(a.codes, a.scale_factors, b.codes, b.scale_factors, m=a.rows, n=b.rows, k=a.k,
                   shift_sum=a.shift + b.shift, snap=snap, alpha=alpha, bias=bias, out_dtype=out_dtype,
                   a_record=a.record, b_record=b.record)
    if kernel_events is not None:
        kernel_events[1].record()
    lib = _native.load()
    tail = (a.rows, b.rows, a.k, int(bool(snap)), *_alpha_arguments(alpha, out.device), _native.ptr(bias),
            _native.dtype_code(bias.dtype) if bias is not None else 0, out.data_ptr(),
            _native.dtype_code(out_dtype), b.rows)
    operands = (a.codes.data_ptr(), a.raw_scale_factors.data_ptr(), a.record.data_ptr(),
                b.codes.data_ptr(), b.raw_scale_factors.data_ptr(), b.record.data_ptr())
    with torch.cuda.device(out.device):
        if fallback_mode() == "workspace":
            workspace = _fallback_workspace(out.device, lib.ue5m3_fallback_workspace_bytes(a.rows, b.rows, a.k))
            status = lib.ue5m3_gemm_fp4_fallback_ws(*operands, *tail, workspace.data_ptr(), workspace.numel(),
                                                    gemm_status(out.device).data_ptr(), _native.stream_ptr(out.device))
            _native.check(status, "ue5m3_gemm_fp4_fallback_ws", launches=2)   # decode, then one GEMM launch for all lists
        else:
            status = lib.ue5m3_gemm_fp4_fallback(*operands, *tail, gemm_status(out.device).data_ptr(),
                                                 _native.stream_ptr(out.device))
            _native.check(status, "ue5m3_gemm_fp4_fallback", launches=2)   # one launch per tile width
    if _window_log is not None:
        _window_log.append((a.record, b.record, (a.rows, b.rows, a.k)))
    return out


def encoded_global_alpha(amax_a: Tensor, amax_b: Tensor, target_a: float, target_b: float) -> Tensor:
    """alpha = fl(amax_a*amax_b) / ((Ta*6)*(Tb*6)), evaluated with the very Torch
    expression of backends/triton/quantization.py:412-420 on the device scalars."""

    return (amax_a * amax_b).to(torch.float32) / ((target_a * 6.0) * (target_b * 6.0))


# ---------------------------------------------------------------------------
# Reference-facing entry points (signatures of backends/triton of the reference)
# ---------------------------------------------------------------------------
def _require_operand(tensor: Tensor, *, name: str) -> None:
    """backends/triton/quantization.py:209-221 without the isfinite pass (see _resolve_amax)."""

    if not isinstance(tensor, Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if tensor.ndim != 2:
        raise ValueError(f"{name} must be rank-2")
    if not tensor.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if tensor.dtype not in {torch.bfloat16, torch.float32}:
        raise TypeError(f"{name} must have dtype bfloat16 or float32")
    if not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _resolve_amax(tensor: Tensor, value: Tensor | float | None, *, name: str, operand: str) -> Tensor:
    """backends/triton/quantization.py:224-244.  The operand's own amax is always taken
    (one pass, on the device) because its bit pattern also answers the reference's
    isfinite check (quantization.py:220-221)."""

    own = tensor_amax(tensor).reshape(1)
    if not math.isfinite(float(own.item())):
        raise ValueError(f"{operand} must contain only finite values")
    if value is None:
        return own
    if isinstance(value, bool):
        raise TypeError(f"{name} must be a scalar tensor or real number")
    if isinstance(value, Tensor):
        if value.numel() != 1:
            raise ValueError(f"{name} must contain exactly one value")
        if value.device != tensor.device:
            raise ValueError(f"{name} must be on the same device as its operand")
        if not value.is_floating_point():
            raise TypeError(f"{name} must have a floating-point dtype")
        result = value.detach().to(dtype=torch.float32).reshape(1).contiguous()
    elif isinstance(value, (int, float)):
        result = torch.tensor([float(value)], device=tensor.device, dtype=torch.float32)
    else:
        raise TypeError(f"{name} must be a scalar tensor or real number")
    scalar = float(result.item())
    if not math.isfinite(scalar) or scalar < 0.0:
        raise ValueError(f"{name} must be finite and non-negative")
    return result


def _resolve_bits(operand: Tensor, bits: Tensor | None, *, rounding: RoundingMode,
                  generator: torch.Generator | None, name: str) -> Tensor | None:
    """backends/triton/quantization.py:247-282; uint8 bits are accepted besides int32."""

    if rounding is not RoundingMode.STOCHASTIC_8BIT_MIDPOINT:
        if bits is not None:
            raise ValueError(f"{name} is only valid with stochastic rounding")
        return None
    if bits is None:
        return torch.randint(0, 256, operand.shape, dtype=torch.int32, device=operand.device, generator=generator)
    if not isinstance(bits, Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if bits.shape != operand.shape:
        raise ValueError(f"{name} must have the same shape as its operand")
    if bits.device != operand.device:
        raise ValueError(f"{name} must be on the same device as its operand")
    if bits.dtype not in (torch.int32, torch.uint8):
        raise TypeError(f"{name} must have dtype int32")
    if not bits.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if bits.dtype is torch.int32 and not bool(((bits >= 0) & (bits <= 255)).all()):
        raise ValueError(f"{name} values must be in [0, 255]")
    return bits


def _validate_common(a: Tensor, b: Tensor, block_size, scale_target_a, scale_target_b, two_dimensional_b) -> None:
    if a.device != b.device:
        raise ValueError("a and b must be on the same CUDA device")
    if a.shape[1] != b.shape[0]:
        raise ValueError("a and b have incompatible K dimensions")
    if block_size not in {16, 32}:
        raise ValueError("block_size must be 16 or 32")
    if a.shape[1] == 0 or a.shape[0] == 0 or b.shape[1] == 0:
        raise ValueError("a and b must have non-empty dimensions")
    if a.shape[1] % block_size:
        raise ValueError("K must be divisible by block_size")
    for label, target in (("scale_target_a", scale_target_a), ("scale_target_b", scale_target_b)):
        if not isinstance(target, (int, float)) or isinstance(target, bool):
            raise TypeError(f"{label} must be a real number")
        if not math.isfinite(target) or target <= 0:
            raise ValueError(f"{label} must be finite and positive")
    if not isinstance(two_dimensional_b, bool):
        raise TypeError("two_dimensional_b must be bool")


def fake_quantize_gemm_operands(
    a: Tensor,
    b: Tensor,
    *,
    block_size: int,
    scale_target_a: float = 448.0,
    scale_target_b: float = 448.0,
    tensor_amax_a: Tensor | float | None = None,
    tensor_amax_b: Tensor | float | None = None,
    rounding_a: str | RoundingMode = RoundingMode.TIES_TO_EVEN,
    rounding_b: str | RoundingMode = RoundingMode.TIES_TO_EVEN,
    random_bits_a: Tensor | None = None,
    random_bits_b: Tensor | None = None,
    generator: torch.Generator | None = None,
    two_dimensional_b: bool = False,
    output_domain: str = "decoded",
    output_dtype: torch.dtype | None = None,
) -> tuple[Tensor, Tensor]:
    """Fake-quantize logical GEMM operands ``A[M,K]`` and ``B[K,N]`` along K.

    Same signature, validation and results as the reference's
    backends/triton/quantization.py:293-409.
    """

    _require_operand(a, name="a")
    _require_operand(b, name="b")
    _validate_common(a, b, block_size, scale_target_a, scale_target_b, two_dimensional_b)
    if output_domain not in {"decoded", "encoded"}:
        raise ValueError("output_domain must be 'decoded' or 'encoded'")
    if output_dtype is None:
        output_dtype = a.dtype
    if output_dtype not in {torch.bfloat16, torch.float32}:
        raise TypeError("output_dtype must be torch.bfloat16 or torch.float32")
    if generator is not None and not isinstance(generator, torch.Generator):
        raise TypeError("generator must be a torch.Generator")
    mode_a = normalize_rounding(rounding_a)
    mode_b = normalize_rounding(rounding_b)
    bits_a = _resolve_bits(a, random_bits_a, rounding=mode_a, generator=generator, name="random_bits_a")
    bits_b = _resolve_bits(b, random_bits_b, rounding=mode_b, generator=generator, name="random_bits_b")
    amax_a = _resolve_amax(a, tensor_amax_a, name="tensor_amax_a", operand="a")
    amax_b = _resolve_amax(b, tensor_amax_b, name="tensor_amax_b", operand="b")
    out_a = quantize_packed(
        a, block_size=block_size, blocking=BLOCK_ROW, tensor_amax=amax_a, scale_target=float(scale_target_a),
        rounding=mode_a, random_bits=bits_a, packed=False, fake_domain=output_domain, fake_dtype=output_dtype,
    ).fake
    out_b = quantize_packed(
        b, block_size=block_size, blocking=BLOCK_2D if two_dimensional_b else BLOCK_COL, tensor_amax=amax_b,
        scale_target=float(scale_target_b), rounding=mode_b, random_bits=bits_b, packed=False, packed_t=False,
        fake_domain=output_domain, fake_dtype=output_dtype,
    ).fake
    return out_a, out_b


def issue_rz_bf16_gemm(a: Tensor, b: Tensor, *, snap_to_1_over_1024: bool = False) -> Tensor:
    """BF16 GEMM with an FP32 round-toward-zero add every K=64 (backends/triton/gemm.py:110-160)."""

    if not isinstance(a, Tensor) or not isinstance(b, Tensor):
        raise TypeError("a and b must be torch.Tensor instances")
    if not a.is_cuda or not b.is_cuda:
        raise ValueError("a and b must be CUDA tensors")
    if a.device != b.device:
        raise ValueError("a and b must be on the same CUDA device")
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("a and b must have dtype bfloat16")
    if a.ndim != 2 or b.ndim != 2:
        raise ValueError("a and b must be rank-2")
    if a.shape[1] != b.shape[0]:
        raise ValueError("a and b have incompatible K dimensions")
    if not a.is_contiguous() or not b.is_contiguous():
        raise ValueError("a and b must be contiguous")
    if a.shape[1] % 64:
        raise ValueError("K must be divisible by 64")
    if not isinstance(snap_to_1_over_1024, bool):
        raise TypeError("snap_to_1_over_1024 must be bool")
    m, k = a.shape
    n = b.shape[1]
    if m == 0 or n == 0 or k == 0:
        return torch.empty((m, n), dtype=torch.float32, device=a.device)
    # The kernel wants the reduction axis contiguous in both operands.
    return gemm_issue_rz(a, b.t().contiguous(), snap=snap_to_1_over_1024, out_dtype=torch.float32)


def probe_matched_fp4_gemm(
    a: Tensor,
    b: Tensor,
    *,
    block_size: int,
    scale_target_a: float = 448.0,
    scale_target_b: float = 448.0,
    tensor_amax_a: Tensor | float | None = None,
    tensor_amax_b: Tensor | float | None = None,
    rounding_a: str | RoundingMode = RoundingMode.TIES_TO_EVEN,
    rounding_b: str | RoundingMode = RoundingMode.TIES_TO_EVEN,
    random_bits_a: Tensor | None = None,
    random_bits_b: Tensor | None = None,
    generator: torch.Generator | None = None,
    two_dimensional_b: bool = False,
    snap_to_1_over_1024: bool = True,
) -> Tensor:
    """Quantize (encoded) -> issue-RZ GEMM -> 1/1024 snap -> * alpha, fp32 out.

    Same signature and results as backends/triton/api.py:23-83; the quantizer writes
    B's encoded values transposed (K contiguous) so the GEMM reads both operands K-major.
    """

    _require_operand(a, name="a")
    _require_operand(b, name="b")
    _validate_common(a, b, block_size, scale_target_a, scale_target_b, two_dimensional_b)
    if a.shape[1] % 64:
        raise ValueError("K must be divisible by 64")
    if not isinstance(snap_to_1_over_1024, bool):
        raise TypeError("snap_to_1_over_1024 must be bool")
    mode_a = normalize_rounding(rounding_a)
    mode_b = normalize_rounding(rounding_b)
    bits_a = _resolve_bits(a, random_bits_a, rounding=mode_a, generator=generator, name="random_bits_a")
    bits_b = _resolve_bits(b, random_bits_b, rounding=mode_b, generator=generator, name="random_bits_b")
    amax_a = _resolve_amax(a, tensor_amax_a, name="tensor_amax_a", operand="a")
    amax_b = _resolve_amax(b, tensor_amax_b, name="tensor_amax_b", operand="b")
    alpha = encoded_global_alpha(amax_a, amax_b, float(scale_target_a), float(scale_target_b))
    blocking_b = BLOCK_2D if two_dimensional_b else BLOCK_COL
    if gemm_path() == "fp4":
        op_a = quantize_fp4_operand(a, block_size=block_size, blocking=BLOCK_ROW, transposed=False,
                                    tensor_amax=amax_a, scale_target=float(scale_target_a), rounding=mode_a,
                                    random_bits=bits_a)
        op_b = quantize_fp4_operand(b, block_size=block_size, blocking=blocking_b, transposed=True,
                                    tensor_amax=amax_b, scale_target=float(scale_target_b), rounding=mode_b,
                                    random_bits=bits_b)
        return gemm_fp4_operands(op_a, op_b, snap=snap_to_1_over_1024, alpha=alpha, out_dtype=torch.float32)
    enc_a = quantize_packed(
        a, block_size=block_size, blocking=BLOCK_ROW, tensor_amax=amax_a, scale_target=float(scale_target_a),
        rounding=mode_a, random_bits=bits_a, packed=False, fake_domain="encoded", fake_dtype=torch.bfloat16,
    ).fake
    enc_bt = quantize_packed(
        b, block_size=block_size, blocking=blocking_b, tensor_amax=amax_b,
        scale_target=float(scale_target_b), rounding=mode_b, random_bits=bits_b, packed=False, packed_t=False,
        fake_domain="encoded", fake_dtype=torch.bfloat16, fake=False, fake_t=True,
    ).fake_t
    return gemm_issue_rz(enc_a, enc_bt, snap=snap_to_1_over_1024, alpha=alpha, out_dtype=torch.float32)


__all__ = [
    "BLOCK_2D",
    "BLOCK_COL",
    "BLOCK_ROW",
    "EpilogueAlpha",
    "Fp4Operand",
    "PackedOperand",
    "available",
    "check_gemm_status",
    "dequantize_packed",
    "encoded_global_alpha",
    "fake_quantize_gemm_operands",
    "gemm_fp4",
    "gemm_fp4_operands",
    "gemm_issue_rz",
    "gemm_path",
    "pack_scales",
    "quantize_fp4_operand",
    "new_window_record",
    "place_row_windows",
    "scale_byte_histogram",
    "log_window_records",
    "window_log_summary",
    "poll_gemm_status",
    "gemm_status",
    "issue_rz_bf16_gemm",
    "probe_matched_fp4_gemm",
    "quantize_packed",
    "tensor_amax",
]
