"""Differential test against the REFERENCE's own Triton kernels on the same GPU
(backends/triton/api.py:23-83, quantization.py:293-409, gemm.py:26-160 of the reference).

The reference package is copied, unmodified, into the git-ignored oracle/_ref/src by
oracle/build.py wherever a reference checkout is reachable; it runs in a child process (its
package has the same name as this repository's).  Skipped when the copy or Triton is absent.

What is compared: the fake-quantized operands in both output domains (bit for bit), and the
probe-matched product against BOTH of this repository's GEMM kernels.  The BF16-issue kernel
issues the instruction shape Triton compiles the reference's `tl.dot` to, so it is expected to
agree bit for bit everywhere; the FP4 tensor-core kernel is expected to agree wherever issue
sums are exact (every distribution the benchmark names) and is measured on the wide-range
family."""

from __future__ import annotations

import importlib.util
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from gpu_helpers import random_bits, student_t_dy, to_np, ulp_distance, wide_range

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
REFERENCE_SRC = ROOT / "oracle" / "_ref" / "src"


def _cases() -> dict[str, dict]:
    g = torch.Generator().manual_seed(123)
    cases = {}

    def add(name, a, b, *, block=16, two_d=False, ta=448.0, tb=448.0, sr=False, fp32=False, amax_a=None):
        entry = dict(a=a.float().numpy(), b=b.float().numpy(), meta=np.array([block, two_d, ta, tb, sr], np.float64))
        if sr:
            entry["bits_a"] = random_bits(a.shape, len(cases) + 1, torch.int32).numpy()
        if fp32:
            entry["fp32"] = np.ones(1)
        if amax_a is not None:
            entry["amax_a"] = np.array(amax_a, np.float64)
        cases[name] = entry

    bf = torch.bfloat16
    # forward: N(0,1) activations x N(0, 0.02^2) weights with 2-D tiles (first, small)
    add("fwd_small", torch.randn(128, 256, generator=g).to(bf), (0.02 * torch.randn(256, 192, generator=g)).to(bf),
        two_d=True)
    add("fwd", torch.randn(256, 512, generator=g).to(bf), (0.02 * torch.randn(512, 384, generator=g)).to(bf), two_d=True)
    add("fwd_b32", torch.randn(192, 1024, generator=g).to(bf), (0.02 * torch.randn(1024, 256, generator=g)).to(bf),
        block=32, two_d=True)
    # data gradient: Student-t dY, stochastic with explicit int32 bits, held (stale) amax
    dy = student_t_dy(192, 512, seed=3)
    add("dgrad_sr", dy, (0.02 * torch.randn(512, 384, generator=g)).to(bf), two_d=True, sr=True,
        amax_a=float(dy.float().abs().max()) * 0.9)
    # weight gradient: dY^T at T = 2048 x squared-ReLU activations blocked along the tokens
    add("wgrad_sr", (1e-4 * torch.randn(128, 256, generator=g)).to(bf),
        torch.relu(torch.randn(256, 320, generator=g)).square().to(bf), block=32, ta=2048.0, sr=True)
    # fp32 inputs with outliers (the round-trip configuration)
    x = torch.randn(128, 512, generator=g)
    x = torch.where(torch.rand(128, 512, generator=g) < 0.01, x * 100.0, x)
    add("fp32_outliers", x, 0.02 * torch.randn(512, 256, generator=g), two_d=True, fp32=True)
    # adversarial for accumulation order: per-block magnitudes 2^U{-12..0}
    add("wide", wide_range(128, 512, lo=-12, seed=21).to(bf), wide_range(256, 512, lo=-12, seed=22).to(bf).t().contiguous())
    return cases


@pytest.fixture(scope="module")
def reference_results(tmp_path_factory):
    if not (REFERENCE_SRC / "ue5m3_fp4" / "backends" / "triton" / "api.py").exists():
        pytest.skip("no copy of the reference package under oracle/_ref/src (made by oracle/build.py where a checkout exists)")
    if importlib.util.find_spec("triton") is None:
        pytest.skip("Triton is not installed")
    folder = tmp_path_factory.mktemp("reference_triton")
    cases = _cases()
    flat = {f"{name}.{key}": value for name, entry in cases.items() for key, value in entry.items()}
    np.savez(folder / "cases.npz", **flat)
    env = dict(os.environ, PYTHONPATH=str(REFERENCE_SRC))
    done = subprocess.run([sys.executable, str(ROOT / "oracle" / "reference_triton_runner.py"),
                           str(folder / "cases.npz"), str(folder / "results.npz")],
                          env=env, capture_output=True, text=True, timeout=900)
    if done.returncode != 0:
        pytest.fail("the reference's Triton path did not run:\n" + done.stdout[-2000:] + done.stderr[-4000:])
    return cases, np.load(folder / "results.npz")


def _tensor(entry, key):
    dtype = torch.float32 if "fp32" in entry else torch.bfloat16
    return torch.from_numpy(entry[key]).to(dtype).cuda()


def _kwargs(entry):
    block, two_d, ta, tb, sr = (float(v) for v in entry["meta"])
    kwargs = dict(block_size=int(block), scale_target_a=ta, scale_target_b=tb, two_dimensional_b=bool(two_d))
    if sr:
        kwargs["rounding_a"] = "StochasticFast"
        kwargs["random_bits_a"] = torch.from_numpy(entry["bits_a"]).cuda()
    if "amax_a" in entry:
        kwargs["tensor_amax_a"] = float(entry["amax_a"])
    return kwargs


def test_fake_quantized_operands_equal_the_reference_triton_kernel(reference_results):
    from ue5m3_fp4.backends.triton import fake_quantize_gemm_operands

    cases, ref = reference_results
    for name, entry in cases.items():
        a, b = _tensor(entry, "a"), _tensor(entry, "b")
        for domain in ("encoded", "decoded"):
            qa, qb = fake_quantize_gemm_operands(a, b, output_domain=domain, output_dtype=torch.float32, **_kwargs(entry))
            assert np.array_equal(to_np(qa), ref[f"{name}.{domain}_a"]), (name, domain, "a")
            assert np.array_equal(to_np(qb), ref[f"{name}.{domain}_b"]), (name, domain, "b")


def test_probe_matched_product_against_the_reference_triton_kernel(reference_results, monkeypatch):
    from ue5m3_fp4.backends.triton import probe_matched_fp4_gemm

    cases, ref = reference_results
    report = {}
    for name, entry in cases.items():
        a, b = _tensor(entry, "a"), _tensor(entry, "b")
        expect = ref[f"{name}.product"]
        for path in ("bf16", "fp4"):
            monkeypatch.setenv("UE5M3_GEMM_PATH", path)
            got = to_np(probe_matched_fp4_gemm(a, b, **_kwargs(entry)))
            differing = float((got != expect).mean())
            worst = int(ulp_distance(got, expect).max())
            report[(name, path)] = (differing, worst)
            print(f"vs reference Triton: {name:14s} {path}: differing {differing:.4f}, max ulp {worst}")
            if name != "wide":
                assert differing == 0.0, (name, path, differing, worst)
    # wide-range family: the BF16-issue kernel issues the reference's own instruction shape
    assert report[("wide", "bf16")][0] == 0.0, report[("wide", "bf16")]
