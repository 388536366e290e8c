"""Generate golden fixtures by importing the reference's own Python code.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports ``ue5m3_fp4.formats`` and ``reproduce.diagnostics.numerics`` from that
checkout (CPU only) and writes ``quantize_golden.npz`` and ``gemm_golden.npz``
beside this script.  The fixtures hold seeded inputs and the reference's outputs,
so the oracle and the CUDA kernels can be checked where the reference is absent.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _reference(root: Path):
    sys.path.insert(0, str(root / "src"))
    sys.path.insert(0, str(root))
    import ue5m3_fp4.formats as formats  # noqa: PLC0415
    from reproduce.diagnostics import numerics  # noqa: PLC0415

    return formats, numerics


def _quantize_case(formats, name, x, *, block, two_d, target, rounding, reference, bits):
    """Reference outputs for one case.

    The block quantizer takes a generator but no explicit random bits
    (formats.py:444-449), so stochastic cases compose the scale values from the
    metadata call (independent of payload rounding) with
    ``round_to_format(..., random_bits=...)`` exactly as formats.py:438-450 does.
    """

    ref_arg = None if reference is None else torch.tensor(reference, dtype=torch.float32)
    _, meta = formats.quantize_dequantize_blocks_with_metadata(
        x, block_size=block, scale_format=formats.UE5M3, scale_target=target,
        rounding="ties_to_even", tensor_reference=ref_arg, two_dimensional=two_d,
    )
    scales = meta.block_scale_codes
    if two_d:
        expanded = scales.repeat_interleave(block, 0).repeat_interleave(block, 1)[: x.shape[0], : x.shape[1]]
    else:
        expanded = scales.repeat_interleave(block, 1)[:, : x.shape[1]]
    decode = meta.global_encode_multiplier.reciprocal()
    decoded_scale = expanded * decode
    payload_input = x.float() * torch.reciprocal(decoded_scale)
    payload = formats.round_to_format(
        payload_input, formats.E2M1, rounding=rounding,
        random_bits=None if bits is None else bits.to(torch.int32),
    )
    dequant = payload * decoded_scale
    if bits is None:
        direct = formats.quantize_dequantize_blocks(
            x, block_size=block, scale_format=formats.UE5M3, scale_target=target,
            rounding=rounding, tensor_reference=ref_arg, two_dimensional=two_d,
        )
        assert torch.equal(direct.float(), dequant.to(x.dtype).float()), name
    return {
        f"{name}.x": x.float().numpy(),
        f"{name}.block": np.int64(block),
        f"{name}.two_d": np.int64(two_d),
        f"{name}.target": np.float32(target),
        f"{name}.sr": np.int64(bits is not None),
        f"{name}.amax": meta.tensor_reference.numpy(),
        f"{name}.bits": np.zeros(0, np.uint8) if bits is None else bits.numpy().astype(np.uint8),
        f"{name}.scales": scales.numpy(),
        f"{name}.block_amax": meta.block_amax.numpy(),
        f"{name}.payload": payload.numpy(),
        f"{name}.dequant": dequant.numpy(),
    }


def quantize_fixtures(formats) -> dict[str, np.ndarray]:
    out: dict[str, np.ndarray] = {}
    g = torch.Generator().manual_seed(20260001)

    # Fake-quant round trip shape family: N(0,1) with 1 % outliers x100.
    x = torch.randn(48, 64, generator=g)
    x = torch.where(torch.rand(48, 64, generator=g) < 0.01, x * 100.0, x)
    out.update(_quantize_case(formats, "c1_b16", x, block=16, two_d=False, target=448.0,
                              rounding="ties_to_even", reference=None, bits=None))
    out.update(_quantize_case(formats, "c1_b32", x, block=32, two_d=False, target=448.0,
                              rounding="ties_to_even", reference=None, bits=None))

    # Upstream-gradient family: Student-t(3) * 1e-3 in bf16, stochastic bits, held amax.
    t = torch.distributions.StudentT(3.0)
    torch.manual_seed(0)
    dy = (t.sample((40, 96)) * 1e-3).to(torch.bfloat16)
    bits = torch.randint(0, 256, dy.shape, generator=g, dtype=torch.int32)
    held = float(dy.float().abs().max()) * 0.6  # stale reference: payload saturation exercised
    out.update(_quantize_case(formats, "c2_sr_b16", dy, block=16, two_d=False, target=448.0,
                              rounding="stochastic_8bit_midpoint", reference=held, bits=bits))
    out.update(_quantize_case(formats, "c2_sr_b32_t2048", dy, block=32, two_d=False, target=2048.0,
                              rounding="stochastic_8bit_midpoint", reference=None, bits=bits))

    # Weight family: N(0, 0.02^2), 2-D tiles, ragged edges (zero padded).
    w = (0.02 * torch.randn(50, 72, generator=g)).to(torch.bfloat16)
    out.update(_quantize_case(formats, "w2d_b16", w, block=16, two_d=True, target=448.0,
                              rounding="ties_to_even", reference=None, bits=None))
    out.update(_quantize_case(formats, "w2d_b32", w, block=32, two_d=True, target=448.0,
                              rounding="ties_to_even", reference=None, bits=None))

    # Wide dynamic range per block (scale subnormals, saturation, 0 -> 1 rule).
    wide = torch.randn(32, 128, generator=g) * torch.exp2(
        torch.randint(-30, 1, (32, 8), generator=g).float()
    ).repeat_interleave(16, 1)
    wide[3, 16:32] = 0.0
    out.update(_quantize_case(formats, "wide_b16", wide, block=16, two_d=False, target=448.0,
                              rounding="ties_to_even", reference=None, bits=None))
    bits_w = torch.randint(0, 256, wide.shape, generator=g, dtype=torch.int32)
    out.update(_quantize_case(formats, "wide_sr_b16", wide, block=16, two_d=False, target=448.0,
                              rounding="stochastic_8bit_midpoint", reference=1e-3, bits=bits_w))

    # Values sitting on and around every E2M1 rounding boundary.
    edges = torch.tensor([0.0, 0.25, 0.5, 0.75, 1.0, 1.25, 1.5, 1.75, 2.0, 2.5, 3.0, 3.5, 4.0, 5.0, 6.0, 5.5])
    grid = torch.cat([edges, torch.nextafter(edges, torch.tensor(10.0)), torch.nextafter(edges, torch.tensor(-10.0)).abs(), -edges])
    grid = grid.reshape(4, 16)
    out.update(_quantize_case(formats, "edges_b16", grid, block=16, two_d=False, target=448.0,
                              rounding="ties_to_even", reference=6.0, bits=None))
    return out


def gemm_fixtures(formats, numerics) -> dict[str, np.ndarray]:
    """Issue-RZ accumulation fixtures from the reference's CPU numerics helpers.

    ``accumulate_issue_partials`` (numerics.py:89-113) is fed exact FP32 issue
    partials; its ``rz`` / ``rz_grid`` outputs are the reference answers for the
    cross-issue rule.  Partials are built so that the FP64 detour inside
    ``add_rz_f32`` is exact (magnitudes within 2^29 of each other).
    """

    out: dict[str, np.ndarray] = {}
    g = torch.Generator().manual_seed(20260002)
    partials = torch.randn(64, 12, generator=g) * torch.exp2(torch.randint(-6, 7, (64, 12), generator=g).float())
    reduced = numerics.accumulate_issue_partials(partials.float())
    out["rz.partials"] = partials.float().numpy()
    out["rz.rz"] = reduced["rz"].numpy()
    out["rz.rz_grid"] = reduced["rz_grid"].numpy()
    out["rz.rn"] = reduced["rn"].numpy()
    left = torch.tensor([1.0, 1.0, -1.0, 3.0, 1e8], dtype=torch.float32)
    right = torch.tensor([2.0**-24, -(2.0**-25), 2.0**-25, 2.0**-23, -1.0], dtype=torch.float32)
    out["rz.pair_left"] = left.numpy()
    out["rz.pair_right"] = right.numpy()
    out["rz.pair_sum"] = numerics.add_rz_f32(left, right).numpy()
    snap_in = torch.tensor([0.5 / 1024, 1.5 / 1024, 2.5 / 1024, -0.5 / 1024, 3.25, 1e9, 1.0 / 4096.0], dtype=torch.float32)
    out["snap.in"] = snap_in.numpy()
    out["snap.out"] = numerics.snap_rne(snap_in, 1024).numpy()
    return out


def rht_fixtures(root: Path) -> dict:
    """The TE-settings comparator's fixed-sign B=16 Hadamard transform (nn/linear.py:80-114),
    run on the CPU: seeded inputs and the reference's BF16 outputs."""

    from ue5m3_fp4.nn.linear import _te_settings_rht_last_dim_b16  # noqa: PLC0415

    g = torch.Generator().manual_seed(1234)
    cases = {
        "normal": torch.randn(32, 128, generator=g).to(torch.bfloat16).float(),
        "small": (1e-3 * torch.randn(24, 64, generator=g)).to(torch.bfloat16).float(),
        "outliers": (torch.randn(16, 96, generator=g)
                     * torch.where(torch.rand(16, 96, generator=g) < 0.03, 100.0, 1.0)).to(torch.bfloat16).float(),
        "fp32": torch.randn(8, 64, generator=g),
        "wide": (torch.randn(16, 64, generator=g)
                 * torch.exp2(torch.randint(-12, 1, (16, 64), generator=g).float())).to(torch.bfloat16).float(),
    }
    out = {"names": np.array(sorted(cases))}
    for name, x in cases.items():
        out[f"{name}.x"] = x.numpy()
        out[f"{name}.y"] = _te_settings_rht_last_dim_b16(x).float().numpy()
    return out


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference>")
    root = Path(sys.argv[1])
    formats, numerics = _reference(root)
    np.savez_compressed(HERE / "quantize_golden.npz", **quantize_fixtures(formats))
    np.savez_compressed(HERE / "gemm_golden.npz", **gemm_fixtures(formats, numerics))
    np.savez_compressed(HERE / "rht_golden.npz", **rht_fixtures(root))
    print("wrote", HERE / "quantize_golden.npz", HERE / "gemm_golden.npz", HERE / "rht_golden.npz")


if __name__ == "__main__":
    main()
