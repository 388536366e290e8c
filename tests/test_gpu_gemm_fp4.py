"""The FP4 block-scaled tensor-core GEMM (ue5m3_gemm_fp4) and its scale packer, through the
C ABI: scale-factor layout against a numpy restatement, the window records of scales outside
UE4M3's range and the recomputation they drive (ue5m3_gemm_fp4_fallback[_ws]), bit-exactness
against the oracle on packed operands, equality with the BF16-issue kernel, and the
benchmark shapes on sampled rows x columns."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from gpu_helpers import accumulation_unit, assert_measured_rule, bf16_round, expect_packed, oracle_quantize, random_bits, student_t_dy, to_np, wide_range
from oracle import ue5m3_oracle as o

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def b200():
    from ue5m3_fp4.backends import b200 as module

    assert module.available()
    return module


@pytest.fixture(autouse=True, params=["workspace", "inline"])
def recomputation_mode(request, monkeypatch):
    """Every test runs with both forms of the recomputation pass: operands decoded once into a
    workspace for the TMA-fed issue-RZ kernel (ue5m3_gemm_fp4_fallback_ws, the default) and
    decoded per tile inside the pass's own kernel (ue5m3_gemm_fp4_fallback)."""

    monkeypatch.setenv("UE5M3_FALLBACK", request.param)
    return request.param


def _expected_scale_layout(scales: np.ndarray, rows: int, k: int, block: int, two_d: bool, shift: int,
                           raw: bool = False) -> np.ndarray:
    """The 512-byte atoms: UE4M3 bytes (re-biased, clamped to the normal range, 1.0 = 0x38 in the
    padding rows) or, with ``raw``, the unmodified UE5M3 bytes (0 = immaterial in the padding rows)."""

    tiles, atoms = (rows + 127) // 128, k // 64
    out = np.full((tiles, atoms, 512), 0 if raw else 0x38, np.uint8)
    group = block if two_d else 1
    for r in range(rows):
        tile, r1, r0 = r // 128, (r % 128) // 32, r % 32
        for h in range(k // 16):
            code = int(scales[r // group, h // (block // 16)])
            if not raw:
                code = min(max(code - ((8 + shift) << 3), 8), 0x7E)
            out[tile, h // 4, r0 * 16 + r1 * 4 + h % 4] = code
    return out.reshape(-1)


@pytest.mark.parametrize("rows,k,block,two_d,shift", [(128, 64, 16, False, 0), (300, 256, 16, False, 1),
                                                      (200, 128, 32, False, 0), (160, 192, 16, True, 3),
                                                      (96, 128, 32, True, 0)])
def test_scale_packer_layout_and_rebias(b200, rows, k, block, two_d, shift):
    g = torch.Generator().manual_seed(rows + k)
    shape = ((rows + block - 1) // block if two_d else rows, k // block)
    lo = (9 + shift) << 3
    scales = torch.randint(lo, lo + 100, shape, generator=g, dtype=torch.int32).to(torch.uint8)
    got, raw, record = b200.pack_scales(scales.cuda(), rows=rows, k=k, block_size=block, two_dimensional=two_d,
                                        shift=shift, want_raw=True)
    assert np.array_equal(to_np(got), _expected_scale_layout(scales.numpy(), rows, k, block, two_d, shift))
    assert np.array_equal(to_np(raw), _expected_scale_layout(scales.numpy(), rows, k, block, two_d, shift, raw=True))
    assert record[:2].tolist() == [0, 0]


def test_scale_window_record(b200):
    """Which UE5M3 bytes fit UE4M3's normal range at shift 0, and what the record then holds."""

    dev = torch.device("cuda", 0)
    for code, outside in [(0x78, 0), ((9 << 3), 0), ((9 << 3) - 1, 1), ((23 << 3) | 6, 0), ((23 << 3) | 7, 1),
                          (0xF7, 1), (1, 1)]:
        scales = torch.full((128, 4), 0x78, dtype=torch.uint8, device=dev)
        scales[5, 1] = code
        scales[77, 0] = code
        scales[77, 3] = code
        _, _, record = b200.pack_scales(scales, rows=128, k=64, block_size=16, two_dimensional=False, shift=0,
                                        want_raw=True)
        rec = record.tolist()
        flags = rec[4 + b200.FALLBACK_MAX_ROWS:4 + b200.FALLBACK_MAX_ROWS + 128]
        if outside:
            assert rec[0] == 2 and rec[1] == 3, hex(code)
            assert [i for i, f in enumerate(flags) if f] == [5, 77]
        else:
            assert rec[0] == 0 and rec[1] == 0 and not any(rec[4:]), hex(code)


def _case(b200, a, bt, *, block, two_d, ta=448.0, tb=448.0, sr=False, held=1.0, seed=0):
    """Quantize packed, run the FP4 GEMM and the BF16-issue GEMM, return both and the oracle."""

    dev = torch.device("cuda", 0)
    bits = random_bits(a.shape, seed, torch.uint8) if sr else None
    amax_a = float(a.float().abs().max()) * held
    amax_b = float(bt.float().abs().max())
    ta_t = torch.tensor([amax_a], device=dev)
    tb_t = torch.tensor([amax_b], device=dev)
    op_a = b200.quantize_fp4_operand(a.cuda(), block_size=block, blocking=b200.BLOCK_ROW, transposed=False,
                                     tensor_amax=ta_t, scale_target=ta, rounding="StochasticFast" if sr else "TTE",
                                     random_bits=None if bits is None else bits.cuda(),
                                     shift_headroom=1 if held < 1.0 else 0)  # stale amax: scales exceed T
    op_b = b200.quantize_fp4_operand(bt.cuda(), block_size=block, blocking=b200.BLOCK_2D if two_d else b200.BLOCK_ROW,
                                     transposed=False, tensor_amax=tb_t, scale_target=tb)
    alpha = b200.encoded_global_alpha(ta_t, tb_t, ta, tb)
    got = b200.gemm_fp4_operands(op_a, op_b, snap=True, alpha=alpha)
    torch.cuda.synchronize()
    b200.check_gemm_status(dev)
    qa = oracle_quantize(a.float(), block=block, blocking=o.BLOCK_ROW, amax=amax_a, target=ta, sr=sr, bits=bits)
    qb = oracle_quantize(bt.float(), block=block, blocking=o.BLOCK_2D if two_d else o.BLOCK_ROW, amax=amax_b, target=tb)
    expect = o.gemm_issue_rz(qa["encoded"], qb["encoded"], snap=True, alpha_value=float(alpha.item()))
    return to_np(got), expect


@pytest.mark.parametrize("block", [16, 32])
@pytest.mark.parametrize("m,k,n", [(35, 128, 69), (128, 64, 256), (300, 320, 520), (256, 4096, 384)])
def test_fp4_gemm_forward_distribution_bit_exact(b200, block, m, k, n):
    g = torch.Generator().manual_seed(m + n)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16)
    got, expect = _case(b200, x, w, block=block, two_d=True)
    assert np.array_equal(got, expect)


def test_fp4_gemm_backward_distributions_bit_exact(b200):
    g = torch.Generator().manual_seed(4)
    dy = student_t_dy(192, 512, seed=3)
    wt = (0.02 * torch.randn(384, 512, generator=g)).to(torch.bfloat16)
    got, expect = _case(b200, dy, wt, block=16, two_d=True, sr=True, held=0.9, seed=5)
    assert np.array_equal(got, expect)
    dyt = (1e-4 * torch.randn(96, 256, generator=g)).to(torch.bfloat16)
    xt = torch.relu(torch.randn(320, 256, generator=g)).square().to(torch.bfloat16)
    got, expect = _case(b200, dyt, xt, block=32, two_d=False, ta=2048.0, sr=True, seed=6)
    assert np.array_equal(got, expect)


def test_fp4_gemm_wide_range_is_the_measured_rule_and_close_to_the_model(b200):
    """Per-block magnitudes over 2^-12..1: issue sums no longer fit fp32 exactly, so the rounding
    inside an issue is visible.  The kernel equals c <- RTZ(c + exact issue sum) bit for bit
    (tests/test_gpu_fp4_accumulation.py pins that rule); against the reference's two-rounding
    model every output stays within one ulp per issue of the largest magnitude ITS accumulation
    passes through."""

    a = wide_range(128, 512, lo=-12, seed=21).to(torch.bfloat16)
    b = wide_range(256, 512, lo=-12, seed=22).to(torch.bfloat16)
    got, expect = _case(b200, a, b, block=16, two_d=False)
    amax_a, amax_b = float(a.float().abs().max()), float(b.float().abs().max())
    qa = oracle_quantize(a.float(), block=16, blocking=o.BLOCK_ROW, amax=amax_a)
    qb = oracle_quantize(b.float(), block=16, blocking=o.BLOCK_ROW, amax=amax_b)
    alpha = o.alpha(np.float32(amax_a), np.float32(amax_b), 448.0, 448.0, reciprocal_form=True)
    native = o.gemm_issue_rz(qa["encoded"], qb["encoded"], snap=True, alpha_value=alpha, native_rule=True)
    unit = accumulation_unit(qa["encoded"], qb["encoded"]) * alpha
    assert_measured_rule(got, native, unit, exact=False)
    ratio = np.abs(got.astype(np.float64) - expect.astype(np.float64)) / unit
    print("fp4 wide-range: differing from the model", float((got != expect).mean()), "max units", float(ratio.max()))
    assert ratio.max() <= 512 // 64 + 1  # one per issue, one for the final scaling by alpha


def test_probe_matched_falls_back_when_a_scale_leaves_the_window(b200, monkeypatch):
    from ue5m3_fp4.backends.triton import probe_matched_fp4_gemm

    g = torch.Generator().manual_seed(9)
    a = torch.randn(64, 128, generator=g)
    a[:, 64:80] *= 2.0**-20  # one block per row far below the UE4M3 window
    a = a.to(torch.bfloat16)
    b = torch.randn(128, 96, generator=g).to(torch.bfloat16)
    results = {}
    for path in ("fp4", "bf16"):
        monkeypatch.setenv("UE5M3_GEMM_PATH", path)
        results[path] = probe_matched_fp4_gemm(a.cuda(), b.cuda(), block_size=16)
    torch.cuda.synchronize()
    assert torch.equal(results["fp4"], results["bf16"])
    qa = oracle_quantize(a.float(), block=16, blocking=o.BLOCK_ROW, amax=float(a.float().abs().max()))
    assert (qa["scale_codes"] < (9 << 3)).any()  # the case does leave the window


def test_fp4_gemm_benchmark_shape_sampled(b200):
    g = torch.Generator().manual_seed(0)
    m, k, n = 8192, 4096, 21504
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16)
    dev = torch.device("cuda", 0)
    xc, wc = x.cuda(), w.cuda()
    ax, aw = b200.tensor_amax(xc).reshape(1), b200.tensor_amax(wc).reshape(1)
    op_a = b200.quantize_fp4_operand(xc, block_size=16, blocking=b200.BLOCK_ROW, transposed=False, tensor_amax=ax,
                                     scale_target=448.0)
    op_b = b200.quantize_fp4_operand(wc, block_size=16, blocking=b200.BLOCK_2D, transposed=False, tensor_amax=aw,
                                     scale_target=448.0)
    alpha = b200.encoded_global_alpha(ax, aw, 448.0, 448.0)
    y = b200.gemm_fp4_operands(op_a, op_b, snap=True, alpha=alpha, out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    b200.check_gemm_status(dev)
    assert op_a.window_counts() == (0, 0) and op_b.window_counts() == (0, 0)
    rows = torch.tensor([0, 1, 127, 128, 4095, 4096, 8063, 8191] + list(range(3000, 3024)))
    col_bands = [0, 240, 256, 10752, 21232, 21488, 7008, 7024]  # whole 16-row bands of W (2-D tiles)
    cols = torch.cat([torch.arange(c, c + 16) for c in col_bands])
    qx = oracle_quantize(x[rows].float(), block=16, blocking=o.BLOCK_ROW, amax=float(ax.item()))
    enc_w = np.concatenate([
        oracle_quantize(w[c:c + 16].float(), block=16, blocking=o.BLOCK_2D, amax=float(aw.item()))["encoded"]
        for c in col_bands
    ])
    expect = o.gemm_issue_rz(qx["encoded"], enc_w, snap=True, alpha_value=float(alpha.item()))
    got = to_np(y[rows.cuda()][:, cols.cuda()])
    assert np.array_equal(got, bf16_round(expect))


@pytest.mark.parametrize("rows,k,block,blocking,sr,dtype", [
    (128, 64, 16, "row", False, torch.bfloat16),
    (300, 256, 16, "row", True, torch.bfloat16),
    (77, 128, 32, "row", False, torch.float32),
    (160, 192, 16, "2d", False, torch.bfloat16),
    (203, 320, 16, "2d", True, torch.float32),
    (96, 128, 32, "2d", False, torch.bfloat16),
    (1000, 1024, 32, "2d", True, torch.bfloat16),
])
def test_one_pass_operand_quantizer_equals_quantize_then_pack(b200, rows, k, block, blocking, sr, dtype):
    """ue5m3_quantize_fp4_operand (codes + UE4M3 atoms in one launch) against ue5m3_quantize
    followed by ue5m3_pack_scales_ue4m3, and its codes and raw scales against the oracle."""

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(rows * 7 + k)
    x = torch.randn(rows, k, generator=g)
    x = x.to(torch.bfloat16).float() if dtype is torch.bfloat16 else x
    bits = random_bits((rows, k), rows + k, torch.uint8) if sr else None
    amax = torch.tensor([float(x.abs().max())], device=dev)
    code = b200.BLOCK_ROW if blocking == "row" else b200.BLOCK_2D
    rounding = "StochasticFast" if sr else "TTE"
    xd = x.to(dtype).cuda()
    bd = None if bits is None else bits.cuda()
    shift = b200.scale_shift_for_target(448.0)
    (op, raw) = b200._quantize_fp4_operand_fused(xd, block, code, amax, 448.0, rounding, bd, shift, want_scales=True)
    two = b200.quantize_packed(xd, block_size=block, blocking=code, tensor_amax=amax, scale_target=448.0,
                               rounding=rounding, random_bits=bd, packed=True, packed_t=False)
    sf, sf_raw, _ = b200.pack_scales(two.scales, rows=rows, k=k, block_size=block, two_dimensional=blocking == "2d",
                                     shift=shift, want_raw=True)
    assert op.window_counts() == (0, 0)
    assert torch.equal(op.codes, two.codes)
    assert torch.equal(raw, two.scales)
    assert torch.equal(op.scale_factors, sf)
    assert torch.equal(op.raw_scale_factors, sf_raw)
    ref = expect_packed(oracle_quantize(x, block=block, blocking=code, amax=float(amax.item()), target=448.0,
                                        sr=sr, bits=bits))
    assert np.array_equal(to_np(op.codes), ref["codes"])
    assert np.array_equal(to_np(raw), ref["scales"])


def test_one_pass_operand_quantizers_fill_the_window_record(b200):
    dev = torch.device("cuda", 0)
    x = torch.ones(192, 128, dtype=torch.bfloat16, device=dev)
    x[5, 3] = 3.0e4  # the scale of every block of ones falls below the UE4M3 window
    x[:, 32:48] = 1.0e3  # except in this band of columns (and the block that holds the maximum)
    amax = torch.tensor([3.0e4], device=dev)
    op = b200.quantize_fp4_operand(x, block_size=16, blocking=b200.BLOCK_ROW, transposed=False, tensor_amax=amax,
                                   scale_target=448.0)
    assert op.window_counts() == (192, 192 * 7 - 1)
    assert op.flagged_rows() == list(range(192))
    # the transposed operand [128, 192]: blocks along the 192 rows of x; only columns 32..47 stay inside
    op_t = b200.quantize_fp4_operand(x, block_size=16, blocking=b200.BLOCK_COL, transposed=True, tensor_amax=amax,
                                     scale_target=448.0)
    listed, units = op_t.window_counts()
    assert listed == 112 and units == 112 * 12 - 1
    assert op_t.flagged_rows() == [c for c in range(128) if not 32 <= c < 48]
    # placement: column 3 holds the tensor maximum next to ones (its scales span the window: listed);
    # every other flagged column is small as a whole and gets a window of its own
    b200.place_row_windows(op_t, None)
    listed_rows, placed = op_t.placement()
    assert listed_rows == [3] and sorted(placed) == [c for c in range(128) if not 32 <= c < 48 and c != 3]
    assert len(set(placed.values())) == 1 and next(iter(placed.values())) < -8
    # the row-blocked operand: every row holds both the 1.0e3 band and blocks of ones -> in range of one
    # window of its own, except row 5 with the 3.0e4 element
    b200.place_row_windows(op, None)
    listed_rows, placed = op.placement()
    assert listed_rows == [5] and sorted(placed) == [r for r in range(192) if r != 5]


def _bf16_path_product(b200, a, bt, *, block, two_d, amax_a, amax_b, monkeypatch):
    from ue5m3_fp4.backends.triton import probe_matched_fp4_gemm

    monkeypatch.setenv("UE5M3_GEMM_PATH", "bf16")
    out = probe_matched_fp4_gemm(a.cuda(), bt.t().contiguous().cuda(), block_size=block, tensor_amax_a=amax_a,
                                 tensor_amax_b=amax_b, two_dimensional_b=two_d)
    monkeypatch.setenv("UE5M3_GEMM_PATH", "fp4")
    return out


@pytest.mark.parametrize("m,k,n,block,two_d,out_dtype", [
    (300, 256, 520, 16, False, torch.float32),
    (300, 256, 520, 16, False, torch.bfloat16),
    (256, 512, 384, 32, True, torch.float32),
    (77, 128, 1030, 16, False, torch.bfloat16),
])
def test_rows_and_columns_outside_the_scale_window_are_recomputed(b200, monkeypatch, m, k, n, block, two_d, out_dtype):
    """A few operand rows of A and of B carry blocks 2^-20 below the rest: their scales leave the
    UE4M3 window, the records list them, and after ue5m3_gemm_fp4_fallback the whole output
    equals the BF16-issue product of the same operands bit for bit."""

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g)
    bt = torch.randn(n, k, generator=g)
    rows_a = sorted({0, 31, min(130, m - 2), m - 1})
    for r in rows_a:
        a[r, 64:64 + block] *= 2.0 ** -20
    a = a.to(torch.bfloat16)
    if two_d:
        bands_b = [1, (n // block) - 1]
        for band in bands_b:
            bt[band * block:(band + 1) * block, 2 * block:3 * block] *= 2.0 ** -20
        rows_b = [r for band in bands_b for r in range(band * block, (band + 1) * block)]
    else:
        rows_b = [3, 255, 256, n - 2]
        for r in rows_b:
            bt[r, 0:block] *= 2.0 ** -20
    bt = bt.to(torch.bfloat16)
    amax_a = torch.tensor([float(a.float().abs().max())], device=dev)
    amax_b = torch.tensor([float(bt.float().abs().max())], device=dev)
    op_a = b200.quantize_fp4_operand(a.cuda(), block_size=block, blocking=b200.BLOCK_ROW, transposed=False,
                                     tensor_amax=amax_a, scale_target=448.0)
    op_b = b200.quantize_fp4_operand(bt.cuda(), block_size=block, blocking=b200.BLOCK_2D if two_d else b200.BLOCK_ROW,
                                     transposed=False, tensor_amax=amax_b, scale_target=448.0)
    assert op_a.flagged_rows() == rows_a and op_b.flagged_rows() == sorted(rows_b)
    alpha = b200.encoded_global_alpha(amax_a, amax_b, 448.0, 448.0)
    bias = torch.randn(n, generator=g).cuda()
    # the FP4 kernel alone gets the flagged rows and columns wrong ...
    alone = b200.gemm_fp4(op_a.codes, op_a.scale_factors, op_b.codes, op_b.scale_factors, m=m, n=n, k=k,
                          shift_sum=op_a.shift + op_b.shift, snap=True, alpha=alpha, bias=bias, out_dtype=out_dtype)
    got = b200.gemm_fp4_operands(op_a, op_b, snap=True, alpha=alpha, bias=bias, out_dtype=out_dtype)
    # these rows mix blocks 2^-20 apart: no window of their own fits, all of them are listed
    assert op_a.placement() == (rows_a, {}) and op_b.placement() == (sorted(rows_b), {})
    torch.cuda.synchronize()
    b200.check_gemm_status(dev)
    expect = (_bf16_path_product(b200, a, bt, block=block, two_d=two_d, amax_a=amax_a, amax_b=amax_b,
                                 monkeypatch=monkeypatch) + bias).to(out_dtype)
    assert torch.equal(got, expect)
    wrong = (alone != expect)
    assert wrong.any()
    keep_rows = torch.ones(m, dtype=torch.bool, device=dev)
    keep_rows[rows_a] = False
    keep_cols = torch.ones(n, dtype=torch.bool, device=dev)
    keep_cols[rows_b] = False
    assert not wrong[keep_rows][:, keep_cols].any()  # ... and nothing else


def test_an_overflowing_window_record_recomputes_the_whole_product(b200, monkeypatch):
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(12)
    m, k, n = 4352, 128, 300
    a = torch.randn(m, k, generator=g)
    a[:, 16:32] *= 2.0 ** -22  # every row: more rows than a record lists
    a = a.to(torch.bfloat16)
    bt = torch.randn(n, k, generator=g).to(torch.bfloat16)
    amax_a = torch.tensor([float(a.float().abs().max())], device=dev)
    amax_b = torch.tensor([float(bt.float().abs().max())], device=dev)
    op_a = b200.quantize_fp4_operand(a.cuda(), block_size=16, blocking=b200.BLOCK_ROW, transposed=False,
                                     tensor_amax=amax_a, scale_target=448.0)
    op_b = b200.quantize_fp4_operand(bt.cuda(), block_size=16, blocking=b200.BLOCK_ROW, transposed=False,
                                     tensor_amax=amax_b, scale_target=448.0)
    assert op_a.window_counts() == (m, m)
    alpha = b200.encoded_global_alpha(amax_a, amax_b, 448.0, 448.0)
    got = b200.gemm_fp4_operands(op_a, op_b, snap=True, alpha=alpha)
    assert op_a.record[2].item() == m  # every row's own scales span the window: all listed, more than fit
    torch.cuda.synchronize()
    b200.check_gemm_status(dev)
    expect = _bf16_path_product(b200, a, bt, block=16, two_d=False, amax_a=amax_a, amax_b=amax_b, monkeypatch=monkeypatch)
    assert torch.equal(got, expect)


def test_alpha_formed_in_the_epilogue_equals_the_aten_expression(b200):
    """EpilogueAlpha (two amax scalars + the fp32 reciprocal, combined inside the kernels)
    against the explicit alpha tensor of backends/triton/quantization.py:412-420, on both GEMM
    kernels and through the recomputation pass."""

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(77)
    a = torch.randn(160, 256, generator=g)
    a[3, 32:48] *= 2.0 ** -21      # one listed row, so that the recomputation pass writes too
    a = a.to(torch.bfloat16).cuda()
    bt = (0.02 * torch.randn(300, 256, generator=g)).to(torch.bfloat16).cuda()
    for ta, tb in ((448.0, 448.0), (2048.0, 448.0)):
        amax_a, amax_b = b200.tensor_amax(a).reshape(1) * 1.37, b200.tensor_amax(bt).reshape(1)
        explicit = b200.encoded_global_alpha(amax_a, amax_b, ta, tb)
        fused = b200.EpilogueAlpha.of(amax_a, amax_b, ta, tb)
        op_a = b200.quantize_fp4_operand(a, block_size=16, blocking=b200.BLOCK_ROW, transposed=False, tensor_amax=amax_a,
                                         scale_target=ta, shift_headroom=1)
        op_b = b200.quantize_fp4_operand(bt, block_size=16, blocking=b200.BLOCK_2D, transposed=False, tensor_amax=amax_b,
                                         scale_target=tb)
        assert op_a.window_counts()[0] == 1
        one = b200.gemm_fp4_operands(op_a, op_b, snap=True, alpha=explicit, out_dtype=torch.bfloat16)
        assert op_a.placement()[0] == [3]
        two = b200.gemm_fp4_operands(op_a, op_b, snap=True, alpha=fused, out_dtype=torch.bfloat16)
        assert torch.equal(one, two)
        enc_a = b200.quantize_packed(a, block_size=16, tensor_amax=amax_a, scale_target=ta, packed=False,
                                     fake_domain="encoded", fake_dtype=torch.bfloat16).fake
        enc_b = b200.quantize_packed(bt, block_size=16, blocking=b200.BLOCK_2D, tensor_amax=amax_b, scale_target=tb,
                                     packed=False, packed_t=False, fake_domain="encoded", fake_dtype=torch.bfloat16).fake
        one = b200.gemm_issue_rz(enc_a, enc_b, snap=True, alpha=explicit)
        two = b200.gemm_issue_rz(enc_a, enc_b, snap=True, alpha=fused)
        assert torch.equal(one, two)
    torch.cuda.synchronize()
    b200.check_gemm_status(dev)


def test_small_rows_get_a_scale_window_of_their_own(b200, monkeypatch):
    """Rows (tokens) of A and rows (output columns) of B that are small as a WHOLE - every block
    2^-18 .. 2^-22 below the tensor's largest - leave the tensor's window but fit one placed at
    their own largest scale: nothing is listed, the FP4 kernel computes them, the epilogue undoes
    the per-row powers of two, and the result equals the BF16-issue product bit for bit."""

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(31)
    m, k, n = 384, 512, 640
    a = torch.randn(m, k, generator=g)
    bt = torch.randn(n, k, generator=g)
    small_a = [1, 64, 200, 383]
    small_b = [0, 127, 128, 300, 639]
    for i, r in enumerate(small_a):
        a[r] *= 2.0 ** -(18 + i)
    for i, r in enumerate(small_b):
        bt[r] *= 2.0 ** -(19 + (i % 3))
    a[7, 0:16] = 0.0   # an all-zero block in a placed-free row and ...
    a[64, 32:48] = 0.0  # ... in a small row: its scale must not anchor the row's window
    a, bt = a.to(torch.bfloat16), bt.to(torch.bfloat16)
    amax_a = torch.tensor([float(a.float().abs().max())], device=dev)
    amax_b = torch.tensor([float(bt.float().abs().max())], device=dev)
    for out_dtype in (torch.float32, torch.bfloat16):
        op_a = b200.quantize_fp4_operand(a.cuda(), block_size=16, blocking=b200.BLOCK_ROW, transposed=False,
                                         tensor_amax=amax_a, scale_target=448.0, shift_headroom=1)
        op_b = b200.quantize_fp4_operand(bt.cuda(), block_size=16, blocking=b200.BLOCK_ROW, transposed=False,
                                         tensor_amax=amax_b, scale_target=448.0)
        assert op_a.flagged_rows() == small_a and op_b.flagged_rows() == small_b
        alpha = b200.EpilogueAlpha.of(amax_a, amax_b, 448.0, 448.0)
        bias = torch.randn(n, generator=g).cuda()
        got = b200.gemm_fp4_operands(op_a, op_b, snap=True, alpha=alpha, bias=bias, out_dtype=out_dtype)
        torch.cuda.synchronize()
        b200.check_gemm_status(dev)
        listed_a, placed_a = op_a.placement()
        listed_b, placed_b = op_b.placement()
        assert listed_a == [] and listed_b == [] and sorted(placed_a) == small_a and sorted(placed_b) == small_b
        assert all(-24 <= shift <= -16 for shift in list(placed_a.values()) + list(placed_b.values()))
        expect = (_bf16_path_product(b200, a, bt, block=16, two_d=False, amax_a=amax_a, amax_b=amax_b,
                                     monkeypatch=monkeypatch) + bias).to(out_dtype)
        assert torch.equal(got, expect)


def _listed(op) -> list[int]:
    return op.placement()[0]


def test_squared_relu_down_proj_at_block_16_forward(b200):
    """Y = X W^T of an MLP down-projection at its training size: X = relu(z)^2 [8192, 21504], B = 16.
    A few dozen blocks of X have scales below the UE4M3 window (all sixteen z nearly zero or
    negative); their rows are listed, recomputed, and, like the other sampled rows, equal the
    oracle bit for bit."""

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(0)
    m, k, n = 8192, 21504, 4096
    x = torch.relu(torch.randn(m, k, generator=g)).square().to(torch.bfloat16)
    w = (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16)
    xc, wc = x.cuda(), w.cuda()
    ax, aw = b200.tensor_amax(xc).reshape(1), b200.tensor_amax(wc).reshape(1)
    op_a = b200.quantize_fp4_operand(xc, block_size=16, blocking=b200.BLOCK_ROW, transposed=False, tensor_amax=ax,
                                     scale_target=448.0, shift_headroom=1)
    op_b = b200.quantize_fp4_operand(wc, block_size=16, blocking=b200.BLOCK_2D, transposed=False, tensor_amax=aw,
                                     scale_target=448.0, shift_headroom=1)
    alpha = b200.encoded_global_alpha(ax, aw, 448.0, 448.0)
    y = b200.gemm_fp4_operands(op_a, op_b, snap=True, alpha=alpha, out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    b200.check_gemm_status(dev)
    listed, placed = op_a.placement()
    flagged = op_a.flagged_rows()
    print("squared-ReLU forward: rows flagged", len(flagged), "placed", len(placed), "listed", len(listed),
          "units outside", op_a.window_counts()[1])
    assert 0 < len(flagged) <= 4096 and op_b.window_counts() == (0, 0) and sorted(listed + list(placed)) == flagged
    qx_all = oracle_quantize(x[flagged].float(), block=16, blocking=o.BLOCK_ROW, amax=float(ax.item()))
    assert (qx_all["scale_codes"] < (10 << 3)).any(axis=1).all()  # every flagged row does leave the tensor's window
    rows = torch.tensor(sorted(set(listed[:16] + sorted(placed)[:16] + [0, 127, 128, 4096, 8191])))
    col_bands = [0, 256, 2048, 4080]
    cols = torch.cat([torch.arange(c, c + 16) for c in col_bands])
    qx = oracle_quantize(x[rows].float(), block=16, blocking=o.BLOCK_ROW, amax=float(ax.item()))
    enc_w = np.concatenate([
        oracle_quantize(w[c:c + 16].float(), block=16, blocking=o.BLOCK_2D, amax=float(aw.item()))["encoded"]
        for c in col_bands
    ])
    expect = bf16_round(o.gemm_issue_rz(qx["encoded"], enc_w, snap=True, alpha_value=float(alpha.item())))
    got = to_np(y[rows.cuda()][:, cols.cuda()])
    assert np.array_equal(got, expect)


def test_squared_relu_down_proj_at_block_16_weight_gradient_operand(b200):
    """dW = dY^T X of the same layer: the operand X^T is blocked along the tokens, so the blocks
    below the window now sit in operand rows that are output COLUMNS; they are listed in B's
    record and recomputed."""

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(1)
    tokens, in_f, out_f = 8192, 21504, 1024
    x = torch.relu(torch.randn(tokens, in_f, generator=g)).square().to(torch.bfloat16)
    dy = (1e-4 * torch.randn(tokens, out_f, generator=g)).to(torch.bfloat16)
    xc, dyc = x.cuda(), dy.cuda()
    ax, ady = b200.tensor_amax(xc).reshape(1), b200.tensor_amax(dyc).reshape(1)
    op_a = b200.quantize_fp4_operand(dyc, block_size=16, blocking=b200.BLOCK_COL, transposed=True, tensor_amax=ady,
                                     scale_target=448.0, shift_headroom=1)
    op_b = b200.quantize_fp4_operand(xc, block_size=16, blocking=b200.BLOCK_COL, transposed=True, tensor_amax=ax,
                                     scale_target=448.0, shift_headroom=1)
    alpha = b200.encoded_global_alpha(ady, ax, 448.0, 448.0)
    dw = b200.gemm_fp4_operands(op_a, op_b, snap=True, alpha=alpha, out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    b200.check_gemm_status(dev)
    listed, placed = op_b.placement()
    flagged = op_b.flagged_rows()
    print("squared-ReLU weight gradient: columns flagged", len(flagged), "placed", len(placed), "listed", len(listed),
          "units outside", op_b.window_counts()[1])
    assert 0 < len(flagged) <= 4096 and op_a.window_counts() == (0, 0) and sorted(listed + list(placed)) == flagged
    cols = torch.tensor(sorted(set(listed[:16] + sorted(placed)[:16] + [0, 255, 256, 21503])))
    rows = torch.tensor([0, 1, 127, 128, 511, 1023])
    q_dy = oracle_quantize(dy[:, rows].float(), block=16, blocking=o.BLOCK_COL, amax=float(ady.item()))
    q_x = oracle_quantize(x[:, cols].float(), block=16, blocking=o.BLOCK_COL, amax=float(ax.item()))
    expect = bf16_round(o.gemm_issue_rz(np.ascontiguousarray(q_dy["encoded"].T), np.ascontiguousarray(q_x["encoded"].T),
                                        snap=True, alpha_value=float(alpha.item())))
    got = to_np(dw[rows.cuda()][:, cols.cuda()])
    assert np.array_equal(got, expect)


@pytest.mark.parametrize("m,k,n,block,two_d", [(256, 256, 256, 16, True), (35, 128, 69, 16, True),
                                               (640, 4096, 768, 16, True), (300, 576, 520, 32, False)])
def test_cta_pair_kernel_is_bit_equal_to_the_single_cta_kernel_and_the_oracle(b200, monkeypatch, m, k, n, block, two_d):
    """UE5M3_FP4_CTA_PAIR=1 selects the cluster-of-two kernel (256 x 256 tiles, cta_group::2)."""

    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    bt = (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16)
    monkeypatch.setenv("UE5M3_FP4_CTA_PAIR", "1")
    pair, expect = _case(b200, a, bt, block=block, two_d=two_d)
    monkeypatch.setenv("UE5M3_FP4_CTA_PAIR", "0")
    single, _ = _case(b200, a, bt, block=block, two_d=two_d)
    assert np.array_equal(pair, single)
    assert np.array_equal(pair, expect)


@pytest.mark.parametrize("k,rows,block,blocking,sr,dtype", [
    (128, 64, 16, "col", False, torch.bfloat16),
    (320, 200, 16, "col", True, torch.bfloat16),
    (256, 77, 32, "col", False, torch.float32),
    (192, 160, 16, "2d", False, torch.bfloat16),
    (448, 300, 16, "2d", False, torch.float32),
    (128, 96, 32, "2d", False, torch.bfloat16),
    (1024, 1000, 32, "col", True, torch.bfloat16),
    (320, 208, 16, "col", True, torch.bfloat16),
    (1024, 1024, 32, "col", True, torch.bfloat16),
    (256, 160, 16, "col", True, torch.float32),
    (64, 16, 16, "2d", True, torch.bfloat16),
    (4096, 1152, 16, "2d", False, torch.bfloat16),
])
def test_one_pass_transposed_operand_equals_quantize_then_pack(b200, k, rows, block, blocking, sr, dtype):
    """ue5m3_quantize_fp4_operand_t (operand = x^T: codes_t + UE4M3 atoms in one launch) against
    ue5m3_quantize with transposed outputs followed by ue5m3_pack_scales_ue4m3."""

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(rows * 5 + k)
    x = torch.randn(k, rows, generator=g)  # x is [K, rows]: the operand is its transpose
    x = x.to(torch.bfloat16).float() if dtype is torch.bfloat16 else x
    bits = random_bits((k, rows), rows + k, torch.uint8) if sr else None
    amax = torch.tensor([float(x.abs().max())], device=dev)
    code = b200.BLOCK_COL if blocking == "col" else b200.BLOCK_2D
    rounding = "StochasticFast" if sr else "TTE"
    xd = x.to(dtype).cuda()
    bd = None if bits is None else bits.cuda()
    shift = b200.scale_shift_for_target(448.0)
    op = b200.quantize_fp4_operand(xd, block_size=block, blocking=code, transposed=True, tensor_amax=amax,
                                   scale_target=448.0, rounding=rounding, random_bits=bd)
    two = b200.quantize_packed(xd, block_size=block, blocking=code, tensor_amax=amax, scale_target=448.0,
                               rounding=rounding, random_bits=bd, packed=False, packed_t=True)
    sf, sf_raw, _ = b200.pack_scales(two.scales_t, rows=rows, k=k, block_size=block, two_dimensional=blocking == "2d",
                                     shift=shift, want_raw=True)
    assert op.window_counts() == (0, 0)
    assert (op.rows, op.k) == (rows, k)
    assert torch.equal(op.codes, two.codes_t)
    assert torch.equal(op.scale_factors, sf)
    assert torch.equal(op.raw_scale_factors, sf_raw)


@pytest.mark.parametrize("k,rows,sr,dtype,wide", [(128, 64, False, torch.bfloat16, False), (320, 208, True, torch.bfloat16, False),
                                                   (256, 160, False, torch.float32, False), (1024, 384, True, torch.bfloat16, False),
                                                   (256, 128, False, torch.bfloat16, True)])
def test_hadamard_transformed_operand_against_the_oracle(b200, k, rows, sr, dtype, wide):
    """TE-settings comparator: the weight-gradient operand x^T with the fixed-sign B=16 Hadamard
    transform along the reduction axis, its D=1 amax and its quantization, against the oracle
    (transform pinned to the reference's function, then the block quantizer)."""

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(k + rows)
    x = torch.randn(k, rows, generator=g) * (1e-3 if sr else 1.0)
    if wide:
        x = wide_range(k, rows, lo=-10, seed=4)
    x = x.to(torch.bfloat16).float() if dtype is torch.bfloat16 else x
    xt_rht = o.rht_b16(np.ascontiguousarray(x.numpy().T))          # [rows, k], transformed along k
    expect_amax = float(np.abs(xt_rht).max())
    xd = x.to(dtype).cuda()
    amax = b200.hadamard_amax_transposed(xd)
    bits = random_bits((k, rows), k * 3 + rows, torch.uint8) if sr else None
    op = b200.quantize_fp4_operand(xd, block_size=16, blocking=b200.BLOCK_COL, transposed=True, tensor_amax=amax,
                                   scale_target=448.0, rounding="StochasticFast" if sr else "TTE",
                                   random_bits=None if bits is None else bits.cuda(), hadamard=True)
    torch.cuda.synchronize()
    # the oracle quantizes the transformed tensor row-wise; its bits are those of x^T
    ref = expect_packed(oracle_quantize(torch.from_numpy(xt_rht), block=16, blocking=o.BLOCK_ROW, amax=expect_amax,
                                        target=448.0, sr=sr, bits=None if bits is None else bits.t().contiguous()))
    if wide:
        # FP32 butterflies instead of an exact sum: allowed to differ where 16 values span many binades
        assert abs(float(amax.item()) - expect_amax) <= 2.0 ** -7 * expect_amax
        assert float((to_np(op.codes) != ref["codes"]).mean()) < 0.01
        return
    assert float(amax.item()) == expect_amax
    assert np.array_equal(to_np(op.codes), ref["codes"])
    shift = b200.scale_shift_for_target(448.0)
    sf = b200.pack_scales(torch.from_numpy(ref["scales"]).cuda(), rows=rows, k=k, block_size=16, two_dimensional=False,
                          shift=shift)
    assert torch.equal(op.scale_factors, sf)


def test_launches_after_a_recorded_failure_mark_their_output(b200):
    """A GEMM launch that finds a failure in the status word does no work; it must not leave the
    output looking like a result.  The failure is written by the host here (nothing waits, nothing
    faults): every element of both kernels' outputs is NaN, including ragged edges, and the host
    check raises and clears the word."""

    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator().manual_seed(5)
    a = torch.randn(300, 256, generator=g).to(torch.bfloat16).cuda()
    bt = torch.randn(200, 256, generator=g).to(torch.bfloat16).cuda()
    amax = torch.ones(1, device=dev) * 8.0
    op_a = b200.quantize_fp4_operand(a, block_size=16, blocking=b200.BLOCK_ROW, transposed=False, tensor_amax=amax,
                                     scale_target=448.0)
    op_b = b200.quantize_fp4_operand(bt, block_size=16, blocking=b200.BLOCK_ROW, transposed=False, tensor_amax=amax,
                                     scale_target=448.0)
    torch.cuda.synchronize()
    b200.check_gemm_status(dev)
    words = b200.gemm_status(dev)
    words.copy_(torch.tensor([1, 99, 7, 3], dtype=torch.int32))
    try:
        for out_dtype in (torch.float32, torch.bfloat16):
            got_fp4 = b200.gemm_fp4_operands(op_a, op_b, snap=True, out_dtype=out_dtype)
            got_rz = b200.gemm_issue_rz(a, bt, snap=True, out_dtype=out_dtype)
            torch.cuda.synchronize()
            assert got_fp4.shape == got_rz.shape == (300, 200)
            assert bool(torch.isnan(got_fp4).all()) and bool(torch.isnan(got_rz).all())
        with pytest.raises(RuntimeError, match="site 99"):
            b200.check_gemm_status(dev)
    finally:
        words.zero_()
    healthy = b200.gemm_fp4_operands(op_a, op_b, snap=True)
    torch.cuda.synchronize()
    b200.check_gemm_status(dev)
    assert bool(torch.isfinite(healthy).all())


def test_workspace_form_checks_its_workspace(b200):
    """ue5m3_gemm_fp4_fallback_ws: the size function is (2 x list capacity + M + N) rows of K bf16
    values, and a workspace that is missing, too small or misaligned is refused before anything
    is launched."""

    from ue5m3_fp4 import _native as native

    lib = native.load()
    m, n, k = 192, 320, 256
    need = lib.ue5m3_fallback_workspace_bytes(m, n, k)
    assert need == (2 * b200.FALLBACK_MAX_ROWS + m + n) * k * 2 == b200.fallback_workspace_bytes(m, n, k)
    assert b200.reserve_fallback_workspace(torch.device("cuda", torch.cuda.current_device()), need) >= need
    assert lib.ue5m3_fallback_workspace_bytes(0, n, k) == 0
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator().manual_seed(3)
    amax = torch.ones(1, device=dev) * 8.0
    ops = [b200.quantize_fp4_operand(torch.randn(r, k, generator=g).to(torch.bfloat16).cuda(), block_size=16,
                                     blocking=b200.BLOCK_ROW, transposed=False, tensor_amax=amax, scale_target=448.0)
           for r in (m, n)]
    out = torch.zeros(m, n, device=dev)
    workspace = torch.empty(need + 16, dtype=torch.uint8, device=dev)

    def call(ws_ptr, ws_bytes):
        a, b = ops
        return lib.ue5m3_gemm_fp4_fallback_ws(
            a.codes.data_ptr(), a.raw_scale_factors.data_ptr(), a.record.data_ptr(), b.codes.data_ptr(),
            b.raw_scale_factors.data_ptr(), b.record.data_ptr(), m, n, k, 1, None, None, None, 0.0, None, 0,
            out.data_ptr(), 1, n, ws_ptr, ws_bytes, None, native.stream_ptr(dev))

    assert call(None, need) == 1                               # invalid argument
    assert call(workspace.data_ptr(), need - 1) == 1
    assert call(workspace.data_ptr() + 8, need) == 4           # alignment
    assert call(workspace.data_ptr(), need) == 0               # empty records: two launches that return at once
    torch.cuda.synchronize()
    assert not out.any()


def test_recomputation_walks_more_tiles_than_there_are_sms(b200, monkeypatch):
    """Every row of A listed (five row tiles) against 10240 columns, and some hundred rows of B
    listed as well: each persistent CTA of the recomputation pass walks several tiles, of two
    products, with an odd number of K=64 issues per tile - so the running issue counter has to
    carry the pipeline's barrier phases from tile to tile.  Equal, bit for bit, to the BF16-issue
    product of the same operands."""

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(21)
    m, k, n = 640, 192, 10240
    a = torch.randn(m, k, generator=g)
    a[:, 32:48] *= 2.0 ** -22            # every row of A spans more than the window
    a = a.to(torch.bfloat16)
    bt = torch.randn(n, k, generator=g)
    bt[::31, 64:80] *= 2.0 ** -22        # 331 rows of B as well
    bt = bt.to(torch.bfloat16)
    amax_a = torch.tensor([float(a.float().abs().max())], device=dev)
    amax_b = torch.tensor([float(bt.float().abs().max())], device=dev)
    op_a = b200.quantize_fp4_operand(a.cuda(), block_size=16, blocking=b200.BLOCK_ROW, transposed=False,
                                     tensor_amax=amax_a, scale_target=448.0)
    op_b = b200.quantize_fp4_operand(bt.cuda(), block_size=16, blocking=b200.BLOCK_ROW, transposed=False,
                                     tensor_amax=amax_b, scale_target=448.0)
    alpha = b200.encoded_global_alpha(amax_a, amax_b, 448.0, 448.0)
    got = b200.gemm_fp4_operands(op_a, op_b, snap=True, alpha=alpha)
    torch.cuda.synchronize()
    b200.check_gemm_status(dev)
    assert op_a.record[2].item() == m and op_b.record[2].item() == len(range(0, n, 31))
    expect = _bf16_path_product(b200, a, bt, block=16, two_d=False, amax_a=amax_a, amax_b=amax_b, monkeypatch=monkeypatch)
    assert torch.equal(got, expect)
