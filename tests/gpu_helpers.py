"""Helpers shared by the GPU parity tests: seeded inputs of the benchmark's value
distributions and oracle-side restatements of the packed layouts."""

from __future__ import annotations

import numpy as np
import torch

from oracle import ue5m3_oracle as o


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy() if t.is_floating_point() else t.detach().cpu().numpy()


def student_t_dy(rows: int, cols: int, seed: int = 0) -> torch.Tensor:
    """Upstream-gradient stand-in: Student-t(3) * 1e-3, rounded to bf16."""

    g = torch.Generator().manual_seed(seed)
    z = torch.randn(rows, cols, generator=g)
    chi = torch.randn(3, rows, cols, generator=g).square().sum(0)
    return (z / torch.sqrt(chi / 3.0) * 1e-3).to(torch.bfloat16)


def outlier_normal(rows: int, cols: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    return torch.where(torch.rand(rows, cols, generator=g) < 0.01, x * 100.0, x)


def wide_range(rows: int, cols: int, lo: int, seed: int = 0, block: int = 16) -> torch.Tensor:
    """randn * 2^U{lo..0} per block: adversarial for accumulation order."""

    g = torch.Generator().manual_seed(seed)
    e = torch.randint(lo, 1, (rows, cols // block), generator=g).float()
    return torch.randn(rows, cols, generator=g) * torch.exp2(e).repeat_interleave(block, 1)


def random_bits(shape, seed: int, dtype=torch.uint8) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 256, tuple(shape), generator=g, dtype=torch.int32).to(dtype)


def oracle_quantize(x: torch.Tensor, *, block, blocking, amax, target=448.0, sr=False, bits=None):
    return o.quantize(
        to_np(x), block=block, blocking=blocking, amax_value=float(amax), target=target,
        rounding=o.ROUND_SR if sr else o.ROUND_TTE, rbits=None if bits is None else to_np(bits).astype(np.uint8),
    )


def expect_packed(q: dict) -> dict:
    """Oracle outputs re-laid as the C ABI lays them out (natural and transposed)."""

    return {
        "codes": o.pack_nibbles(q["nibbles"]),
        "codes_t": o.pack_nibbles(np.ascontiguousarray(q["nibbles"].T)),
        "scales": q["scale_codes"],
        "scales_t": np.ascontiguousarray(q["scale_codes"].T),
    }


def bf16_round(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).float().numpy()


def ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in fp32 units in the last place between two finite fp32 arrays."""

    def key(v):
        i = np.ascontiguousarray(v, dtype=np.float32).view(np.int32).astype(np.int64)
        return np.where(i < 0, -(i & 0x7FFFFFFF), i)

    return np.abs(key(a) - key(b))


def accumulation_unit(enc_a: np.ndarray, enc_bt: np.ndarray, group: int = 64) -> np.ndarray:
    """Per output, one fp32 ulp of the largest magnitude its accumulation passes through: the
    sums of each ``group`` of consecutive reduction elements (64 = one issue, 16 = one BF16
    tensor-core instruction), the running sum inside an issue and the running sum across
    issues (float64 estimates).  Deviations between accumulation rules are stated in this unit."""

    a = np.asarray(enc_a, dtype=np.float64)
    b = np.asarray(enc_bt, dtype=np.float64)
    k = a.shape[1]
    largest = np.zeros((a.shape[0], b.shape[0]))
    total = np.zeros_like(largest)
    for issue in range(0, k, 64):
        inside = np.zeros_like(largest)
        for g in range(issue, issue + 64, group):
            part = a[:, g:g + group] @ b[:, g:g + group].T
            inside += part
            largest = np.maximum(largest, np.maximum(np.abs(part), np.abs(inside)))
        total += inside
        largest = np.maximum(largest, np.abs(total))
    return np.spacing(largest.astype(np.float32)).astype(np.float64)


def assert_measured_rule(got: np.ndarray, native: np.ndarray, unit: np.ndarray, *, exact: bool) -> float:
    """``got`` against the oracle's statement of the FP4 instruction's accumulation.  Where all
    addends of every issue lie well inside the instruction's alignment window the two must be
    equal (``exact``); on the extreme families a handful of outputs per million sit on the
    window's edge, which the oracle states to within a bit: at most 1e-4 of the outputs may
    differ, each by at most one unit.  Returns the differing fraction."""

    differing = float((got != native).mean())
    if exact:
        assert differing == 0.0, differing
        return differing
    assert differing <= 1e-4, differing
    assert np.all(np.abs(got.astype(np.float64) - native.astype(np.float64)) <= unit)
    return differing
