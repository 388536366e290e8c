"""GPU parity of the issue-RZ GEMM and of the full probe-matched composition against the
oracle (exact K=64 partials, RNE; RTZ across issues; RNE 1/1024 snap; alpha).

Bit-exact wherever the 64 products of an issue sum without rounding in fp32 (all the
benchmark's operand distributions); the wide-dynamic-range family, where the tensor core's
own intra-issue accumulation is observable, is checked to a stated tolerance."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from gpu_helpers import (accumulation_unit, bf16_round, oracle_quantize, outlier_normal, random_bits, student_t_dy, to_np,
                         ulp_distance, wide_range)
from oracle import ue5m3_oracle as o

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def b200():
    from ue5m3_fp4.backends import b200 as module

    assert module.available()
    return module


def _healthy(b200):
    torch.cuda.synchronize()
    b200.check_gemm_status(torch.device("cuda", torch.cuda.current_device()))


def _small_ints(rows, cols, seed, step):
    g = torch.Generator().manual_seed(seed)
    return (torch.randint(-12, 13, (rows, cols), generator=g).float() * step).to(torch.bfloat16)


@pytest.mark.parametrize("m,k,n", [(32, 64, 64), (33, 128, 67), (128, 256, 256), (600, 128, 700), (257, 1024, 513)])
def test_issue_rz_exact_on_exactly_summable_operands(b200, m, k, n):
    from ue5m3_fp4.backends.triton import issue_rz_bf16_gemm

    a = _small_ints(m, k, m + k, 0.5)
    b = _small_ints(k, n, n + k, 0.25)
    raw = issue_rz_bf16_gemm(a.cuda(), b.cuda())
    snapped = issue_rz_bf16_gemm(a.cuda(), b.cuda(), snap_to_1_over_1024=True)
    _healthy(b200)
    assert raw.shape == (m, n) and raw.dtype is torch.float32
    assert torch.equal(snapped, torch.round(raw * 1024.0) / 1024.0)  # reference tests/test_triton_gemm.py:24-32
    expect = o.gemm_issue_rz(to_np(a), to_np(b).T, snap=False)
    assert np.array_equal(to_np(raw), expect)


def test_issue_rz_round_toward_zero_between_issues(b200):
    """Per-issue partials exact, cross-issue sums inexact: only the RTZ rule decides."""

    g = torch.Generator().manual_seed(7)
    m, n, issues = 128, 256, 24
    a = torch.zeros(m, issues * 64)
    b = torch.zeros(issues * 64, n)
    # one product per issue: a power-of-two-scaled 8-bit integer pair -> partial exact
    for j in range(issues):
        a[:, j * 64 + (j % 64)] = torch.randint(-127, 128, (m,), generator=g).float() * 2.0 ** ((j * 5) % 23 - 11)
        b[j * 64 + (j % 64), :] = torch.randint(-127, 128, (n,), generator=g).float()
    a, b = a.to(torch.bfloat16), b.to(torch.bfloat16)
    from ue5m3_fp4.backends.triton import issue_rz_bf16_gemm

    got = issue_rz_bf16_gemm(a.cuda(), b.cuda())
    _healthy(b200)
    expect = o.gemm_issue_rz(to_np(a), to_np(b).T, snap=False)
    rn = to_np(a).astype(np.float64) @ to_np(b).astype(np.float64)
    assert np.array_equal(to_np(got), expect)
    assert (expect != rn.astype(np.float32)).mean() > 0.05  # the family does exercise RTZ


def test_issue_rz_rejects_wrong_k_and_dtype(b200):
    from ue5m3_fp4.backends.triton import issue_rz_bf16_gemm

    a = torch.ones((2, 65), device="cuda", dtype=torch.bfloat16)
    b = torch.ones((65, 2), device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="divisible by 64"):
        issue_rz_bf16_gemm(a, b)
    with pytest.raises(TypeError, match="bfloat16"):
        issue_rz_bf16_gemm(a.float(), b.float())


def test_alpha_is_the_reference_expression_on_cuda_tensors(b200):
    """ATen divides a CUDA tensor by a host scalar as a multiplication by its fp32 reciprocal;
    the oracle's default alpha form restates that."""

    for ta, tb, va, vb in [(448.0, 448.0, 4.5, 0.094), (2048.0, 448.0, 1.3e-3, 7.1), (448.0, 448.0, 3.0, 3.0)]:
        aa = torch.tensor([va], device="cuda")
        ab = torch.tensor([vb], device="cuda")
        ref = b200.encoded_global_alpha(aa, ab, ta, tb)
        assert ref.item() == o.alpha(float(aa.item()), float(ab.item()), ta, tb, reciprocal_form=True)


def _probe_case(b200, a, b, *, block, two_d, ta=448.0, tb=448.0, sr_a=False, amax_a=None, amax_b=None, seed=0):
    from ue5m3_fp4.backends.triton import probe_matched_fp4_gemm

    bits_a = random_bits(a.shape, seed, torch.int32) if sr_a else None
    amax_a = float(a.float().abs().max()) if amax_a is None else amax_a
    amax_b = float(b.float().abs().max()) if amax_b is None else amax_b
    got = probe_matched_fp4_gemm(
        a.cuda(), b.cuda(), block_size=block, scale_target_a=ta, scale_target_b=tb,
        tensor_amax_a=amax_a, tensor_amax_b=amax_b, rounding_a="StochasticFast" if sr_a else "TTE",
        random_bits_a=None if bits_a is None else bits_a.cuda(), two_dimensional_b=two_d,
    )
    _healthy(b200)
    qa = oracle_quantize(a.float(), block=block, blocking=o.BLOCK_ROW, amax=amax_a, target=ta, sr=sr_a, bits=bits_a)
    bt = b.float().t().contiguous()
    qb = oracle_quantize(bt, block=block, blocking=o.BLOCK_2D if two_d else o.BLOCK_ROW, amax=amax_b, target=tb)
    alpha = o.alpha(np.float32(amax_a), np.float32(amax_b), ta, tb, reciprocal_form=True)
    expect = o.gemm_issue_rz(qa["encoded"], qb["encoded"], snap=True, alpha_value=alpha)
    return to_np(got), expect


@pytest.mark.parametrize("block", [16, 32])
@pytest.mark.parametrize("m,k,n", [(35, 128, 69), (256, 512, 320), (128, 4096, 256)])
def test_probe_matched_forward_distribution_is_bit_exact(b200, gemm_path, block, m, k, n):
    g = torch.Generator().manual_seed(m * n)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w_t = (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16).t().contiguous()
    got, expect = _probe_case(b200, x, w_t, block=block, two_d=True)
    assert np.array_equal(got, expect)


def test_probe_matched_backward_distributions_are_bit_exact(b200, gemm_path):
    g = torch.Generator().manual_seed(11)
    # dgrad: dY (Student-t, stochastic, held amax) x W (2-D tiles)
    dy = student_t_dy(192, 512, seed=3)
    w = (0.02 * torch.randn(512, 384, generator=g)).to(torch.bfloat16)
    got, expect = _probe_case(b200, dy, w, block=16, two_d=True, sr_a=True,
                              amax_a=float(dy.float().abs().max()) * 0.9, seed=5)
    assert np.array_equal(got, expect)
    # wgrad: dY^T (stochastic, T=2048) x X (squared-ReLU activations, 1-D blocks along tokens)
    dyt = (1e-4 * torch.randn(96, 256, generator=g)).to(torch.bfloat16)
    x = torch.relu(torch.randn(256, 320, generator=g)).square().to(torch.bfloat16)
    got, expect = _probe_case(b200, dyt, x, block=32, two_d=False, ta=2048.0, sr_a=True, seed=6)
    assert np.array_equal(got, expect)
    # fp32 master weights and outlier activations
    xo = outlier_normal(64, 256, seed=8).to(torch.bfloat16)
    wf = 0.02 * torch.randn(256, 128, generator=g)
    got, expect = _probe_case(b200, xo, wf, block=16, two_d=True)
    assert np.array_equal(got, expect)


def test_wide_dynamic_range_deviation_is_bounded(b200, gemm_path):
    """Per-block magnitudes spanning 2^-12..1: the exact issue sum no longer fits fp32, so the
    tensor core's rounding inside an issue shows against the model's "exact partial, rounded to
    nearest".  Stated tolerance, per output: the deviation is at most c ulps of the largest
    magnitude THAT output's accumulation passes through, c = one per issue (+1 for alpha) for
    the FP4 instruction (one rounding per K=64 issue) and four per issue for the BF16-issue
    kernel (one rounding per K=16 instruction; this kernel equals the reference's own Triton
    kernel bit for bit, tests/test_gpu_reference_triton.py)."""

    a = wide_range(128, 512, lo=-12, seed=21).to(torch.bfloat16)
    b = wide_range(256, 512, lo=-12, seed=22).to(torch.bfloat16).t().contiguous()
    got, expect = _probe_case(b200, a, b, block=16, two_d=False)
    amax_a, amax_b = float(a.float().abs().max()), float(b.float().abs().max())
    qa = oracle_quantize(a.float(), block=16, blocking=o.BLOCK_ROW, amax=amax_a)
    qb = oracle_quantize(b.float().t().contiguous(), block=16, blocking=o.BLOCK_ROW, amax=amax_b)
    alpha = o.alpha(np.float32(amax_a), np.float32(amax_b), 448.0, 448.0, reciprocal_form=True)
    issues = 512 // 64
    group, allowed = (64, issues + 1) if gemm_path == "fp4" else (16, 4 * issues + 1)
    unit = accumulation_unit(qa["encoded"], qb["encoded"], group=group) * alpha
    ratio = np.abs(got.astype(np.float64) - expect.astype(np.float64)) / unit
    print("wide-range", gemm_path, ": differing outputs", float((got != expect).mean()), "max ulp of the output",
          int(ulp_distance(got, expect).max()), "max units", float(ratio.max()))
    assert ratio.max() <= allowed



def test_headline_shape_sampled_tiles(b200):
    """M8192 K4096 N21504 forward GEMM: full-size launch, oracle on sampled rows x columns."""

    from ue5m3_fp4.backends import b200 as ops

    g = torch.Generator().manual_seed(0)
    m, k, n = 8192, 4096, 21504
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16)
    xc, wc = x.cuda(), w.cuda()
    amax_x, amax_w = ops.tensor_amax(xc).reshape(1), ops.tensor_amax(wc).reshape(1)
    xe = ops.quantize_packed(xc, block_size=16, tensor_amax=amax_x, packed=False, fake_domain="encoded",
                             fake_dtype=torch.bfloat16).fake
    we = ops.quantize_packed(wc, block_size=16, blocking=ops.BLOCK_2D, tensor_amax=amax_w, packed=False,
                             packed_t=False, fake_domain="encoded", fake_dtype=torch.bfloat16).fake
    alpha = ops.encoded_global_alpha(amax_x, amax_w, 448.0, 448.0)
    y = ops.gemm_issue_rz(xe, we, snap=True, alpha=alpha, out_dtype=torch.bfloat16)
    _healthy(b200)
    rows = torch.tensor([0, 1, 127, 128, 4095, 4096, 8063, 8191] + list(range(3000, 3024)))
    cols = torch.tensor([0, 255, 256, 511, 10752, 21247, 21248, 21503] + list(range(7000, 7040)))
    expect = o.gemm_issue_rz(to_np(xe[rows.cuda()]), to_np(we[cols.cuda()]), snap=True, alpha_value=float(alpha.item()))
    got = to_np(y[rows.cuda()][:, cols.cuda()])
    assert np.array_equal(got, bf16_round(expect))
    # encoded operands equal the oracle's on the sampled rows (2-D tiles need whole 16-row bands)
    qx = oracle_quantize(x[rows].float(), block=16, blocking=o.BLOCK_ROW, amax=float(amax_x.item()))
    assert np.array_equal(to_np(xe[rows.cuda()]), qx["encoded"])
    qw = oracle_quantize(w[7008:7040].float(), block=16, blocking=o.BLOCK_2D, amax=float(amax_w.item()))
    assert np.array_equal(to_np(we[7008:7040]), qw["encoded"])
