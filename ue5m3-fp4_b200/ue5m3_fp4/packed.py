"""A self-describing container for one packed FP4 tensor: E2M1 nibble codes, UE5M3 block-scale
bytes and what is needed to interpret them (shape, block size and geometry, tensor amax and
scale target).

The reference has no packed form at all - it keeps fake-quantized values and re-quantizes the
weights of a frozen model in every forward pass (nn/linear.py:549-554,710-718 of the
reference).  This is the storable form of what the kernels of this package consume: 0.5 byte
per element plus one byte per block, written once after the post-load lifecycle has frozen a
weight's amax and read back straight into a GEMM operand.

File layout (little endian): the 8 magic bytes ``UE5M3FP4``, a uint64 header length, a UTF-8
JSON header, then the codes and the scale bytes back to back.  Nibble convention and scale
byte as everywhere in this package: element 2j in the low nibble, nibble = sign<<3 | index into
{0,.5,1,1.5,2,3,4,6}; scale byte = E<<3|M with bias 15 (formats.py:114-134 of the reference).
"""

from __future__ import annotations

import json
import struct
from dataclasses import dataclass
from pathlib import Path

import torch
from torch import Tensor

_MAGIC = b"UE5M3FP4"
_VERSION = 1
_BLOCKINGS = {"row": 0, "col": 1, "2d": 2}


@dataclass(slots=True)
class PackedFP4Tensor:
    """``codes`` [rows, ceil(cols/2)] uint8 and ``scales`` uint8 ([rows, ceil(cols/B)] for 1 x B
    blocks, [ceil(rows/B), ceil(cols/B)] for B x B tiles) of a [rows, cols] tensor."""

    codes: Tensor
    scales: Tensor
    rows: int
    cols: int
    block_size: int
    blocking: str            # "row" (1 x B along the last axis) or "2d" (B x B tiles)
    tensor_amax: float
    scale_target: float
    source_dtype: str = "bfloat16"
    name: str = ""

    def __post_init__(self) -> None:
        if self.blocking not in ("row", "2d"):
            raise ValueError("blocking must be 'row' or '2d'")
        if self.block_size not in (16, 32):
            raise ValueError("block_size must be 16 or 32")
        blocks = (self.cols + self.block_size - 1) // self.block_size
        scale_rows = self.rows if self.blocking == "row" else (self.rows + self.block_size - 1) // self.block_size
        if tuple(self.codes.shape) != (self.rows, (self.cols + 1) // 2) or self.codes.dtype is not torch.uint8:
            raise ValueError("codes must be uint8 [rows, ceil(cols/2)]")
        if tuple(self.scales.shape) != (scale_rows, blocks) or self.scales.dtype is not torch.uint8:
            raise ValueError("scales must be uint8 with one byte per block")

    # ------------------------------------------------------------------ building
    @classmethod
    def quantize(cls, tensor: Tensor, *, block_size: int, two_dimensional: bool, tensor_amax: Tensor | float,
                 scale_target: float = 448.0, name: str = "") -> "PackedFP4Tensor":
        """Quantize a rank-2 CUDA tensor (ties to even) with the kernels of this package."""

        from ue5m3_fp4.backends import b200

        if isinstance(tensor_amax, Tensor):
            amax = tensor_amax.detach().to(torch.float32).reshape(1)
        else:
            amax = torch.tensor([float(tensor_amax)], dtype=torch.float32, device=tensor.device)
        packed = b200.quantize_packed(tensor.detach().contiguous(), block_size=block_size,
                                      blocking=b200.BLOCK_2D if two_dimensional else b200.BLOCK_ROW, tensor_amax=amax,
                                      scale_target=scale_target, packed=True, packed_t=False)
        return cls(packed.codes, packed.scales, tensor.shape[0], tensor.shape[1], block_size,
                   "2d" if two_dimensional else "row", float(amax.item()), float(scale_target),
                   str(tensor.dtype).replace("torch.", ""), name)

    # ------------------------------------------------------------------ file form
    def save(self, path: str | Path) -> None:
        header = {
            "format": "ue5m3_fp4_packed_tensor", "version": _VERSION, "name": self.name,
            "rows": self.rows, "cols": self.cols, "block_size": self.block_size, "blocking": self.blocking,
            "payload": "e2m1, two codes per byte, even element in the low nibble",
            "scale": "ue5m3 byte E<<3|M, bias 15", "tensor_amax_fp32_bits": _float_bits(self.tensor_amax),
            "tensor_amax": self.tensor_amax, "scale_target": self.scale_target, "source_dtype": self.source_dtype,
            "codes_bytes": self.codes.numel(), "scales_bytes": self.scales.numel(),
            "scales_shape": list(self.scales.shape),
        }
        blob = json.dumps(header, sort_keys=True).encode()
        with open(path, "wb") as handle:
            handle.write(_MAGIC)
            handle.write(struct.pack("<Q", len(blob)))
            handle.write(blob)
            handle.write(self.codes.detach().cpu().contiguous().numpy().tobytes())
            handle.write(self.scales.detach().cpu().contiguous().numpy().tobytes())

    @classmethod
    def load(cls, path: str | Path, device: torch.device | str = "cpu") -> "PackedFP4Tensor":
        with open(path, "rb") as handle:
            if handle.read(8) != _MAGIC:
                raise ValueError(f"{path} is not a packed UE5M3/FP4 tensor file")
            (length,) = struct.unpack("<Q", handle.read(8))
            header = json.loads(handle.read(length).decode())
            if header.get("format") != "ue5m3_fp4_packed_tensor" or header.get("version") != _VERSION:
                raise ValueError("unsupported packed tensor header")
            codes = bytearray(handle.read(header["codes_bytes"]))
            scales = bytearray(handle.read(header["scales_bytes"]))
        if len(codes) != header["codes_bytes"] or len(scales) != header["scales_bytes"]:
            raise ValueError("packed tensor file is truncated")
        rows, cols = header["rows"], header["cols"]
        codes_t = torch.frombuffer(codes, dtype=torch.uint8).reshape(rows, (cols + 1) // 2).to(device)
        scales_t = torch.frombuffer(scales, dtype=torch.uint8).reshape(header["scales_shape"]).to(device)
        amax = _bits_float(header["tensor_amax_fp32_bits"])
        return cls(codes_t, scales_t, rows, cols, header["block_size"], header["blocking"], amax,
                   float(header["scale_target"]), header.get("source_dtype", "bfloat16"), header.get("name", ""))

    # ------------------------------------------------------------------ use
    def dequantize(self, out_dtype: torch.dtype = torch.float32) -> Tensor:
        """p * (s * dec) (formats.py:439,450 of the reference), on the tensors' CUDA device."""

        from ue5m3_fp4.backends import b200

        amax = torch.tensor([self.tensor_amax], dtype=torch.float32, device=self.codes.device)
        return b200.dequantize_packed(self.codes, self.scales, rows=self.rows, cols=self.cols, block_size=self.block_size,
                                      two_dimensional=self.blocking == "2d", tensor_amax=amax,
                                      scale_target=self.scale_target, out_dtype=out_dtype)

    def gemm_operand(self, *, shift_headroom: int = 0):
        """The K-major operand of the FP4 GEMM (codes as stored, scales re-laid for the tensor
        core); ``cols`` is the reduction axis and must be a multiple of 64."""

        from ue5m3_fp4.backends import b200

        if not self.codes.is_cuda:
            raise RuntimeError("move the packed tensor to a CUDA device first; there is no CPU path")
        if self.cols % 64:
            raise ValueError("the reduction axis must be a multiple of 64")
        shift = b200.scale_shift_for_target(self.scale_target) + shift_headroom
        sf, raw, record = b200.pack_scales(self.scales, rows=self.rows, k=self.cols, block_size=self.block_size,
                                           two_dimensional=self.blocking == "2d", shift=shift, want_raw=True)
        return b200.Fp4Operand(self.codes, sf, shift, self.rows, self.cols, raw, record)

    def to(self, device: torch.device | str) -> "PackedFP4Tensor":
        return PackedFP4Tensor(self.codes.to(device), self.scales.to(device), self.rows, self.cols, self.block_size,
                               self.blocking, self.tensor_amax, self.scale_target, self.source_dtype, self.name)


def _float_bits(value: float) -> int:
    return struct.unpack("<I", struct.pack("<f", value))[0]


def _bits_float(bits: int) -> float:
    return struct.unpack("<f", struct.pack("<I", bits))[0]


__all__ = ["PackedFP4Tensor"]
