"""Format descriptors, rounding-mode names and the packed block quantizer front end.

Mirrors the public names of the reference's ``formats.py`` (format descriptors
formats.py:62-134, rounding aliases formats.py:23-59, block quantizer
formats.py:460-518).  The reference module is a CPU Torch model of VALUES; here the
same functions run on the sm_100a kernels and additionally expose the packed
storage (E2M1 nibbles, UE5M3 scale bytes).  CUDA tensors only; there is no CPU path.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from enum import StrEnum

import torch
from torch import Tensor


class RoundingMode(StrEnum):
    TIES_TO_EVEN = "ties_to_even"
    STOCHASTIC_8BIT_MIDPOINT = "stochastic_8bit_midpoint"


_ALIASES = {
    "tiestoeven": RoundingMode.TIES_TO_EVEN,
    "tte": RoundingMode.TIES_TO_EVEN,
    "stochasticfast": RoundingMode.STOCHASTIC_8BIT_MIDPOINT,
    "stochastic8bitmidpoint": RoundingMode.STOCHASTIC_8BIT_MIDPOINT,
}


def normalize_rounding(rounding: str | RoundingMode) -> RoundingMode:
    """Canonical rounding mode for a documented name or alias (formats.py:41-59)."""

    if isinstance(rounding, RoundingMode):
        return rounding
    if not isinstance(rounding, str):
        raise TypeError("rounding must be a string or RoundingMode")
    key = rounding.strip().replace("-", "_").lower().replace("_", "")
    try:
        return _ALIASES[key]
    except KeyError as error:
        choices = ", ".join(mode.value for mode in RoundingMode)
        raise ValueError(f"unknown rounding mode {rounding!r}; expected {choices}") from error


@dataclass(frozen=True, slots=True)
class FloatFormat:
    """A finite floating-point value set (formats.py:62-111)."""

    name: str
    total_bits: int
    exponent_bits: int
    fraction_bits: int
    exponent_bias: int
    signed: bool
    has_subnormals: bool
    max_finite: float

    def __post_init__(self) -> None:
        if self.total_bits != int(self.signed) + self.exponent_bits + self.fraction_bits:
            raise ValueError("total_bits does not match the format fields")
        if self.exponent_bits <= 0 or self.fraction_bits < 0:
            raise ValueError("format bit counts must be non-negative")
        if self.exponent_bias <= 0 or not math.isfinite(self.max_finite) or self.max_finite <= 0:
            raise ValueError("format bias and maximum must be positive")

    @property
    def precision(self) -> int:
        return self.fraction_bits + 1

    @property
    def smallest_normal(self) -> float:
        return 2.0 ** (1 - self.exponent_bias)

    @property
    def smallest_subnormal(self) -> float:
        if not self.has_subnormals:
            return self.smallest_normal
        return 2.0 ** (1 - self.exponent_bias - self.fraction_bits)


E2M1 = FloatFormat("E2M1", 4, 2, 1, 1, True, True, 6.0)
# The all-ones exponent field is reserved, so the largest finite value is 1.875 * 2^15.
UE5M3 = FloatFormat("UE5M3", 8, 5, 3, 15, False, True, 61_440.0)


@dataclass(frozen=True, slots=True)
class BlockQuantizationMetadata:
    """Scale information of one block quantization (formats.py:276-283), plus packed storage."""

    tensor_reference: Tensor
    global_encode_multiplier: Tensor
    block_scale_codes: Tensor  # real-valued UE5M3 scales, one per block
    block_scale_bytes: Tensor  # the same scales as UE5M3 bytes (E<<3 | M)
    payload_codes: Tensor  # packed E2M1 nibbles, two per byte, even element low


def _check_block_args(tensor: Tensor, block_size: int, scale_format: FloatFormat, scale_target: float) -> None:
    if not isinstance(tensor, Tensor):
        raise TypeError("tensor must be a torch.Tensor")
    if not tensor.is_floating_point():
        raise TypeError("tensor must have a floating-point dtype")
    if tensor.numel() == 0:
        raise ValueError("block quantization requires a non-empty tensor")
    if not tensor.is_cuda:
        raise RuntimeError("the B200 block quantizer requires a CUDA tensor; there is no CPU path")
    if type(block_size) is not int or block_size not in (16, 32):
        raise ValueError("block_size must be 16 or 32")
    if scale_format != UE5M3:
        raise ValueError("scale_format must be UE5M3")
    if (
        type(scale_target) not in (int, float)
        or not math.isfinite(float(scale_target))
        or not float(scale_target) > 0
    ):
        raise ValueError("scale_target must be a finite positive number")


def quantize_dequantize_blocks_with_metadata(
    tensor: Tensor,
    *,
    block_size: int,
    scale_format: FloatFormat,
    scale_target: float,
    rounding: str | RoundingMode,
    generator: torch.Generator | None = None,
    tensor_reference: Tensor | float | None = None,
    two_dimensional: bool = False,
    random_bits: Tensor | None = None,
) -> tuple[Tensor, BlockQuantizationMetadata]:
    """Quantize -> dequantize with packed metadata (formats.py:496-518).

    ``tensor`` is viewed as ``[-1, last]``; 1-D blocks run along the last axis,
    ``two_dimensional=True`` tiles the last two axes of a rank-2 tensor.
    """

    from ue5m3_fp4.backends import b200

    _check_block_args(tensor, block_size, scale_format, scale_target)
    mode = normalize_rounding(rounding)
    if two_dimensional and tensor.ndim != 2:
        raise ValueError("two_dimensional=True requires a rank-2 tensor")
    if tensor.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("tensor must have dtype bfloat16 or float32")
    flat = tensor.reshape(-1, tensor.shape[-1]).contiguous()
    if tensor_reference is None:
        reference = b200.tensor_amax(flat)
        if not bool(torch.isfinite(reference)):
            raise ValueError("tensor must contain only finite values")
    else:
        reference = torch.as_tensor(tensor_reference, dtype=torch.float32, device=tensor.device).reshape(())
        if not bool(torch.isfinite(reference)) or bool(reference < 0):
            raise ValueError("tensor_reference must be finite and non-negative")
    bits = random_bits
    if mode is RoundingMode.STOCHASTIC_8BIT_MIDPOINT and bits is None:
        bits = torch.randint(0, 256, flat.shape, dtype=torch.int32, device=flat.device, generator=generator)
    packed = b200.quantize_packed(
        flat,
        block_size=block_size,
        blocking=b200.BLOCK_2D if two_dimensional else b200.BLOCK_ROW,
        tensor_amax=reference,
        scale_target=float(scale_target),
        rounding=mode,
        random_bits=None if bits is None else bits.reshape(flat.shape),
        fake_domain="dequant",
        fake_dtype=tensor.dtype,
    )
    encode = b200.global_encode_multiplier(reference, float(scale_target))
    metadata = BlockQuantizationMetadata(
        tensor_reference=reference.detach().clone(),
        global_encode_multiplier=encode,
        block_scale_codes=b200.scale_bytes_to_values(packed.scales),
        block_scale_bytes=packed.scales,
        payload_codes=packed.codes,
    )
    return packed.fake.reshape(tensor.shape), metadata


def quantize_dequantize_blocks(tensor: Tensor, **kwargs) -> Tensor:
    """Fake-quantize E2M1 payloads with UE5M3 block scales (formats.py:460-493)."""

    result, _ = quantize_dequantize_blocks_with_metadata(tensor, **kwargs)
    return result


__all__ = [
    "E2M1",
    "UE5M3",
    "BlockQuantizationMetadata",
    "FloatFormat",
    "RoundingMode",
    "normalize_rounding",
    "quantize_dequantize_blocks",
    "quantize_dequantize_blocks_with_metadata",
]
