"""GPU parity of amax / quantize / dequantize against the oracle and the reference
fixtures, through the C ABI (ctypes binding in ue5m3_fp4._native).  Bit-exact."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import golden_case_names
from gpu_helpers import (expect_packed, oracle_quantize, outlier_normal, random_bits, student_t_dy, to_np,
                         wide_range)
from oracle import ue5m3_oracle as o

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def b200():
    from ue5m3_fp4.backends import b200 as module

    assert module.available(), "CUDA device or sm_100a library missing"
    return module


def _amax_t(value: float) -> torch.Tensor:
    return torch.tensor([value], dtype=torch.float32, device="cuda")


def test_e2m1_hardware_conversion_equals_software_rule_for_every_fp32(b200):
    from ue5m3_fp4 import _native

    count = torch.zeros(1, dtype=torch.int64, device="cuda")
    first = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    status = _native.load().ue5m3_test_e2m1_cvt(0, 1 << 32, count.data_ptr(), first.data_ptr(), None)
    _native.check(status, "ue5m3_test_e2m1_cvt")
    torch.cuda.synchronize()
    assert count.item() == 0, f"first differing fp32 pattern: {first.item() & 0xFFFFFFFF:#010x}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,offset", [(1, 0), (7, 0), (4099, 1), (1 << 20, 3), (33554432 + 5, 0)])
def test_amax_matches_and_stays_on_device(b200, dtype, n, offset):
    g = torch.Generator().manual_seed(n)
    host = torch.randn(n + offset, generator=g).to(dtype)
    host[(n + offset) // 2] = -37.5
    x = host.cuda()[offset:]
    got = b200.tensor_amax(x)
    assert got.is_cuda and got.dtype is torch.float32 and got.ndim == 0
    assert got.item() == host[offset:].float().abs().max().item()
    # scratch is left ready: a second call on the same stream gives the same answer
    assert b200.tensor_amax(x).item() == got.item()


def test_amax_flags_non_finite_inputs(b200):
    x = torch.ones(5000, dtype=torch.bfloat16, device="cuda")
    x[1234] = float("inf")
    assert torch.isinf(b200.tensor_amax(x))
    x[77] = float("nan")
    assert torch.isnan(b200.tensor_amax(x))
    y = torch.ones(5000, dtype=torch.float32, device="cuda")
    y[4999] = float("nan")
    assert torch.isnan(b200.tensor_amax(y))


def _check_case(b200, x_host, *, block, blocking, amax, target, sr, bits_host, dtype, bits_dtype=torch.uint8):
    x = x_host.to(dtype).cuda().contiguous()
    bits = None if bits_host is None else bits_host.to(bits_dtype).cuda().contiguous()
    q = oracle_quantize(x, block=block, blocking=blocking, amax=amax, target=target, sr=sr, bits=bits_host)
    exp = expect_packed(q)
    for domain, key in (("encoded", "encoded"), ("decoded", "decoded"), ("dequant", "dequant")):
        got = b200.quantize_packed(
            x, block_size=block, blocking=blocking, tensor_amax=_amax_t(amax), scale_target=target,
            rounding="StochasticFast" if sr else "TTE", random_bits=bits, packed=blocking != b200.BLOCK_COL,
            packed_t=blocking != b200.BLOCK_ROW, fake_domain=domain, fake_dtype=torch.float32,
            fake=True, fake_t=blocking != b200.BLOCK_ROW,
        )
        if got.codes is not None:
            assert np.array_equal(to_np(got.codes), exp["codes"]), "codes"
            assert np.array_equal(to_np(got.scales), exp["scales"]), "scales"
        if got.codes_t is not None:
            assert np.array_equal(to_np(got.codes_t), exp["codes_t"]), "codes_t"
            assert np.array_equal(to_np(got.scales_t), exp["scales_t"]), "scales_t"
        assert np.array_equal(to_np(got.fake), q[key]), domain
        if got.fake_t is not None:
            assert np.array_equal(to_np(got.fake_t), q[key].T), domain + "_t"
    return q


def test_quantizer_reproduces_reference_fixtures(b200, quantize_golden):
    g = quantize_golden
    for name in golden_case_names(g):
        sr = bool(int(g[f"{name}.sr"]))
        x = torch.from_numpy(g[f"{name}.x"])
        bits = torch.from_numpy(g[f"{name}.bits"].astype(np.int32)) if sr else None
        two_d = bool(int(g[f"{name}.two_d"]))
        q = _check_case(
            b200, x, block=int(g[f"{name}.block"]), blocking=b200.BLOCK_2D if two_d else b200.BLOCK_ROW,
            amax=float(g[f"{name}.amax"]), target=float(g[f"{name}.target"]), sr=sr, bits_host=bits,
            dtype=torch.float32,
        )
        assert np.array_equal(q["dequant"], g[f"{name}.dequant"]), name
        assert np.array_equal(o.scale_values(q["scale_codes"]), g[f"{name}.scales"]), name


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("block", [16, 32])
@pytest.mark.parametrize("rows,cols", [(37, 64), (256, 4096), (5, 17), (3, 40), (130, 96)])
def test_row_blocks_ties_to_even(b200, dtype, block, rows, cols):
    x = outlier_normal(rows, cols, seed=rows * cols).to(dtype).float()
    _check_case(b200, x, block=block, blocking=b200.BLOCK_ROW, amax=float(x.abs().max()), target=448.0,
                sr=False, bits_host=None, dtype=dtype)


@pytest.mark.parametrize("bits_dtype", [torch.uint8, torch.int32])
@pytest.mark.parametrize("block,target", [(16, 448.0), (32, 2048.0)])
@pytest.mark.parametrize("rows,cols", [(64, 4096), (33, 48), (7, 160)])
def test_row_blocks_stochastic_with_held_amax(b200, bits_dtype, block, target, rows, cols):
    dy = student_t_dy(rows, cols, seed=cols).float()
    bits = random_bits(dy.shape, seed=rows, dtype=torch.int32)
    held = float(dy.abs().max()) * 0.7  # stale reference: saturating payloads included
    _check_case(b200, dy, block=block, blocking=b200.BLOCK_ROW, amax=held, target=target, sr=True,
                bits_host=bits, dtype=torch.bfloat16, bits_dtype=bits_dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("block", [16, 32])
@pytest.mark.parametrize("rows,cols", [(128, 64), (256, 192), (100, 72), (33, 7), (512, 640)])
def test_column_blocks_and_two_dimensional_tiles(b200, dtype, block, rows, cols):
    g = torch.Generator().manual_seed(rows + cols)
    w = (0.02 * torch.randn(rows, cols, generator=g)).to(dtype).float()
    amax = float(w.abs().max())
    _check_case(b200, w, block=block, blocking=b200.BLOCK_2D, amax=amax, target=448.0, sr=False,
                bits_host=None, dtype=dtype)
    _check_case(b200, w, block=block, blocking=b200.BLOCK_COL, amax=amax, target=448.0, sr=False,
                bits_host=None, dtype=dtype)
    bits = random_bits(w.shape, seed=cols, dtype=torch.int32)
    _check_case(b200, w, block=block, blocking=b200.BLOCK_COL, amax=amax * 0.8, target=2048.0, sr=True,
                bits_host=bits, dtype=dtype)


def test_wide_dynamic_range_scale_subnormals_and_saturation(b200):
    x = wide_range(64, 256, lo=-34, seed=3)
    x[5, 32:48] = 0.0
    x[6] = 0.0
    _check_case(b200, x, block=16, blocking=b200.BLOCK_ROW, amax=float(x.abs().max()), target=448.0, sr=False,
                bits_host=None, dtype=torch.float32)
    _check_case(b200, x, block=16, blocking=b200.BLOCK_ROW, amax=1e-6, target=448.0, sr=True,
                bits_host=random_bits(x.shape, 9, torch.int32), dtype=torch.float32)
    _check_case(b200, torch.zeros(32, 64), block=16, blocking=b200.BLOCK_2D, amax=0.0, target=448.0, sr=False,
                bits_host=None, dtype=torch.float32)


def test_known_answer_operation_order_on_device(b200):
    # reference tests/test_formats.py:161-196 at block 16 (the block is padded with zeros)
    x = torch.zeros(1, 16)
    x[0, 0] = 7.209771652307365e-15
    got = b200.quantize_packed(x.cuda(), block_size=16, tensor_amax=_amax_t(8.30072435974513e-17))
    assert o.scale_values(to_np(got.scales)).item() == 40960.0
    y = torch.zeros(1, 16)
    y[0, 0], y[0, 1] = 2.7757528175464845e-18, 8.410989948970382e-08
    got = b200.quantize_packed(y.cuda(), block_size=16, tensor_amax=_amax_t(4.857566965417253e-19),
                               fake_domain="dequant")
    assert o.scale_values(to_np(got.scales)).item() == 61440.0
    assert got.fake[0, 0].item() == 0.0


def test_dequantize_kernel(b200):
    x = outlier_normal(70, 96, seed=1)
    amax = float(x.abs().max())
    for two_d in (False, True):
        blocking = b200.BLOCK_2D if two_d else b200.BLOCK_ROW
        got = b200.quantize_packed(x.cuda(), block_size=16, blocking=blocking, tensor_amax=_amax_t(amax),
                                   fake_domain="dequant", packed_t=False)
        back = b200.dequantize_packed(got.codes, got.scales, rows=70, cols=96, block_size=16,
                                      two_dimensional=two_d, tensor_amax=_amax_t(amax))
        assert torch.equal(back, got.fake)
        q = oracle_quantize(x, block=16, blocking=blocking, amax=amax)
        assert np.array_equal(to_np(back), q["dequant"])


def test_headline_shape_stochastic_quantize_full_size(b200):
    """bf16 8192 x 4096, B=16, StochasticFast with uint8 bits and a held amax (the quantize
    benchmark's workload): every code, scale byte and dequantized value against the oracle."""

    dy = student_t_dy(8192, 4096, seed=0)
    bits = random_bits(dy.shape, seed=1, dtype=torch.uint8)
    held = float(dy.float().abs().max())
    got = b200.quantize_packed(dy.cuda(), block_size=16, tensor_amax=_amax_t(held), rounding="StochasticFast",
                               random_bits=bits.cuda(), fake_domain="dequant", fake_dtype=torch.float32)
    q = oracle_quantize(dy.float(), block=16, blocking=o.BLOCK_ROW, amax=held, sr=True, bits=bits)
    assert np.array_equal(to_np(got.codes), o.pack_nibbles(q["nibbles"]))
    assert np.array_equal(to_np(got.scales), q["scale_codes"])
    assert np.array_equal(to_np(got.fake), q["dequant"])
    back = b200.dequantize_packed(got.codes, got.scales, rows=8192, cols=4096, block_size=16,
                                  two_dimensional=False, tensor_amax=_amax_t(held))
    assert torch.equal(back, got.fake)


def test_round_trip_configuration_full_size(b200):
    """fp32 4096 x 4096, N(0,1) with a seeded 1 % of the entries multiplied by 100, B=16 along
    the last axis, target 448 from the CURRENT tensor's amax (D=1, taken by ue5m3_amax), ties to
    even: packed nibble codes, UE5M3 scale bytes and the dequantized fp32 tensor, every element
    against the oracle; the packed form alone dequantizes to the same tensor."""

    x = outlier_normal(4096, 4096, seed=0)
    xd = x.cuda()
    amax = b200.tensor_amax(xd).reshape(1)
    assert amax.item() == x.abs().max().item()
    got = b200.quantize_packed(xd, block_size=16, tensor_amax=amax, scale_target=448.0, rounding="TTE",
                               fake_domain="dequant", fake_dtype=torch.float32)
    q = oracle_quantize(x, block=16, blocking=o.BLOCK_ROW, amax=float(amax.item()))
    assert got.codes.shape == (4096, 2048) and got.scales.shape == (4096, 256)
    assert np.array_equal(to_np(got.codes), o.pack_nibbles(q["nibbles"]))
    assert np.array_equal(to_np(got.scales), q["scale_codes"])
    assert np.array_equal(to_np(got.fake), q["dequant"])
    back = b200.dequantize_packed(got.codes, got.scales, rows=4096, cols=4096, block_size=16,
                                  two_dimensional=False, tensor_amax=amax)
    assert torch.equal(back, got.fake)
    # the outliers do stretch the block scales over many binades (UE5M3's reason for being)
    assert int(q["scale_codes"].max()) - int(q["scale_codes"].min()) >= 6 * 8


def test_entry_point_contract_of_the_reference(b200):
    from ue5m3_fp4.backends.triton import fake_quantize_gemm_operands

    a = torch.ones((2, 64), device="cuda", dtype=torch.bfloat16)
    b = torch.ones((64, 2), device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="block_size"):
        fake_quantize_gemm_operands(a, b, block_size=64)
    with pytest.raises(ValueError, match="output_domain"):
        fake_quantize_gemm_operands(a, b, block_size=16, output_domain="packed")
    with pytest.raises(ValueError, match="only valid with stochastic"):
        fake_quantize_gemm_operands(a, b, block_size=16, random_bits_a=torch.zeros_like(a, dtype=torch.int32))
    with pytest.raises(ValueError, match="finite"):
        fake_quantize_gemm_operands(a * float("inf"), b, block_size=16)
    za, zb = fake_quantize_gemm_operands(torch.zeros(3, 64, device="cuda"), torch.zeros(64, 5, device="cuda"),
                                         block_size=16, output_dtype=torch.float32)
    assert za.count_nonzero().item() == 0 and zb.count_nonzero().item() == 0


@pytest.mark.parametrize("block", [16, 32])
@pytest.mark.parametrize("two_d", [False, True])
@pytest.mark.parametrize("domain", ["decoded", "encoded"])
def test_fake_quantize_gemm_operands_against_oracle(b200, block, two_d, domain):
    from ue5m3_fp4.backends.triton import fake_quantize_gemm_operands

    g = torch.Generator().manual_seed(1234)
    a = torch.randn((37, 64), generator=g).to(torch.bfloat16)
    b = torch.randn((64, 71), generator=g).to(torch.bfloat16)
    bits_a = random_bits(a.shape, 1, torch.int32)
    bits_b = random_bits(b.shape, 2, torch.int32)
    out_a, out_b = fake_quantize_gemm_operands(
        a.cuda(), b.cuda(), block_size=block, scale_target_a=2048.0, scale_target_b=448.0,
        rounding_a="StochasticFast", rounding_b="StochasticFast", random_bits_a=bits_a.cuda(),
        random_bits_b=bits_b.cuda(), two_dimensional_b=two_d, output_domain=domain, output_dtype=torch.float32,
    )
    qa = oracle_quantize(a.float(), block=block, blocking=o.BLOCK_ROW, amax=float(a.float().abs().max()),
                         target=2048.0, sr=True, bits=bits_a)
    qb = oracle_quantize(b.float(), block=block, blocking=o.BLOCK_2D if two_d else o.BLOCK_COL,
                         amax=float(b.float().abs().max()), target=448.0, sr=True, bits=bits_b)
    assert np.array_equal(to_np(out_a), qa[domain])
    assert np.array_equal(to_np(out_b), qb[domain])


@pytest.mark.parametrize("rows,cols,block,blocking", [(64, 256, 16, "row"), (37, 160, 32, "row"), (128, 192, 16, "col"),
                                                     (100, 72, 16, "col"), (96, 128, 16, "2d"), (33, 50, 16, "row")])
def test_counter_based_bits_equal_their_materialised_tensor(b200, rows, cols, block, blocking):
    """UE5M3_BITS_PHILOX: the quantizer computes its random bytes; the same call with the
    bytes written out by ue5m3_philox_bytes as an explicit uint8 tensor gives the same bits,
    on the streaming, the ragged and the tile kernels."""

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(rows * cols)
    x = torch.randn(rows, cols, generator=g).to(torch.bfloat16).cuda()
    amax = torch.tensor([float(x.float().abs().max()) * 0.9], device=dev)
    stream = b200.PhiloxBits(torch.tensor([0x1234567 + rows, 77 + cols], dtype=torch.int64, device=dev))
    explicit = stream.materialize((rows, cols))
    code = {"row": b200.BLOCK_ROW, "col": b200.BLOCK_COL, "2d": b200.BLOCK_2D}[blocking]
    kw = dict(block_size=block, blocking=code, tensor_amax=amax, rounding="StochasticFast",
              packed=blocking != "col", packed_t=blocking != "row")
    a = b200.quantize_packed(x, random_bits=stream, **kw)
    b = b200.quantize_packed(x, random_bits=explicit, **kw)
    for name in ("codes", "scales", "codes_t", "scales_t"):
        ta, tb = getattr(a, name), getattr(b, name)
        assert (ta is None) == (tb is None)
        if ta is not None:
            assert torch.equal(ta, tb), name
    other = b200.PhiloxBits(torch.tensor([0x1234567 + rows, 78 + cols], dtype=torch.int64, device=dev))
    assert not torch.equal(other.materialize((rows, cols)), explicit)


def test_counter_based_bits_in_the_one_pass_operand_kernels(b200):
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(192, 256, generator=g).to(torch.bfloat16).cuda()
    amax = torch.tensor([float(x.float().abs().max())], device=dev)
    stream = b200.PhiloxBits(torch.tensor([99, 3], dtype=torch.int64, device=dev))
    explicit = stream.materialize(x.shape)
    for blocking, transposed in [(b200.BLOCK_ROW, False), (b200.BLOCK_COL, True)]:
        kw = dict(block_size=16, blocking=blocking, transposed=transposed, tensor_amax=amax, scale_target=448.0,
                  rounding="StochasticFast")
        a = b200.quantize_fp4_operand(x, random_bits=stream, **kw)
        b = b200.quantize_fp4_operand(x, random_bits=explicit, **kw)
        assert torch.equal(a.codes, b.codes) and torch.equal(a.scale_factors, b.scale_factors)


def test_counter_based_bits_are_uniform_bytes(b200):
    dev = torch.device("cuda", 0)
    stream = b200.PhiloxBits(torch.tensor([42, 7], dtype=torch.int64, device=dev))
    sample = stream.materialize((1 << 22,)).cpu().numpy()
    counts = np.bincount(sample, minlength=256)
    expected = sample.size / 256
    chi2 = float(((counts - expected) ** 2 / expected).sum())
    assert 150.0 < chi2 < 400.0, chi2  # 255 degrees of freedom
    assert abs(float(sample.mean()) - 127.5) < 0.2
    pairs = np.corrcoef(sample[:-1].astype(np.float64), sample[1:].astype(np.float64))[0, 1]
    assert abs(pairs) < 0.005


def test_philox_known_answer(b200):
    """Philox4x32-10 with counter 0 and key 0 (the published known-answer vector)."""

    dev = torch.device("cuda", 0)
    key = torch.tensor([0, 0], dtype=torch.int64, device=dev)
    raw = b200.PhiloxBits(key).materialize((16,)).cpu().numpy()
    assert [int(v) for v in raw.view(np.uint32)] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]


def _philox4x32_10(counter, key):
    """Plain-Python Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3")."""

    c, k = list(counter), list(key)
    for _ in range(10):
        p0, p1 = 0xD2511F53 * c[0], 0xCD9E8D57 * c[2]
        c = [(p1 >> 32) ^ c[1] ^ k[0], p1 & 0xFFFFFFFF, (p0 >> 32) ^ c[3] ^ k[1], p0 & 0xFFFFFFFF]
        k = [(k[0] + 0x9E3779B9) & 0xFFFFFFFF, (k[1] + 0xBB67AE85) & 0xFFFFFFFF]
    return c


def test_philox_stream_definition(b200):
    """byte e of the stream = byte e % 16 of Philox4x32-10(key = seed, counter = {e / 16, stream})."""

    assert _philox4x32_10([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    dev = torch.device("cuda", 0)
    seed, stream = 0x0123456789ABCDEF, 0x0FEDCBA987654321
    key = torch.tensor([seed, stream], dtype=torch.int64, device=dev)
    raw = b200.PhiloxBits(key).materialize((5 * 16 + 7,)).cpu().numpy()
    for unit in range(5):
        words = _philox4x32_10([unit, 0, stream & 0xFFFFFFFF, stream >> 32], [seed & 0xFFFFFFFF, seed >> 32])
        expect = np.array(words, dtype=np.uint32).view(np.uint8)
        assert np.array_equal(raw[16 * unit:16 * unit + 16], expect), unit


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,cols,block", [(128, 128, 16), (192, 320, 16), (448, 64, 32), (256, 384, 32)])
def test_weight_operands_of_both_orientations_from_one_launch(b200, dtype, rows, cols, block):
    """ue5m3_quantize_fp4_operand_both: W and W^T as packed GEMM operands from one read of a weight
    with B x B blocks equal, bit for bit, what the two single-orientation quantizers write -
    codes, tensor-core scale atoms, raw scale atoms and window records, including all-zero blocks
    and blocks whose scale leaves the tensor core's range."""

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(rows + cols + block)
    w = 0.02 * torch.randn(rows, cols, generator=g)
    w[:16, :16] = 0.0                       # an all-zero block
    w[32:64, cols // 2:] *= 2.0 ** -22      # scales far below the window at this shift
    w[5, 3] = 1.5                           # the amax, well above everything else
    w = w.to(dtype).cuda()
    amax = b200.tensor_amax(w).reshape(1)
    both = b200.quantize_fp4_operand_both(w, block_size=block, tensor_amax=amax, scale_target=448.0, shift_headroom=1)
    assert both is not None
    for operand, transposed in zip(both, (False, True)):
        single = b200.quantize_fp4_operand(w, block_size=block, blocking=b200.BLOCK_2D, transposed=transposed,
                                           tensor_amax=amax, scale_target=448.0, shift_headroom=1)
        assert (operand.rows, operand.k, operand.shift) == (single.rows, single.k, single.shift)
        assert torch.equal(operand.codes, single.codes)
        assert torch.equal(operand.scale_factors, single.scale_factors)
        assert torch.equal(operand.raw_scale_factors, single.raw_scale_factors)
        assert operand.window_counts() == single.window_counts() and operand.window_counts()[0] > 0
        assert sorted(operand.flagged_rows()) == sorted(single.flagged_rows())
    assert b200.quantize_fp4_operand_both(w[:, :40].contiguous(), block_size=block, tensor_amax=amax,
                                          scale_target=448.0) is None
