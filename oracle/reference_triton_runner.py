"""Runs the REFERENCE's own Triton kernels on the cases of an .npz file and writes their outputs
to another .npz file.  Test infrastructure: started as a child process by the GPU parity tests,
with PYTHONPATH pointing at oracle/_ref/src (a copy of the reference package that
oracle/build.py places there), so that its `ue5m3_fp4` is the reference and not this
repository's package of the same name.

    python oracle/reference_triton_runner.py cases.npz results.npz

Case keys: `<name>.a` [M,K] and `<name>.b` [K,N] (float32 holding bf16-exact values unless
`<name>.fp32` is set), `<name>.meta` = [block, two_d, target_a, target_b, sr_a] and optionally
`<name>.bits_a` (int32), `<name>.amax_a`, `<name>.amax_b`.  Outputs per case: the encoded and
decoded fake-quantized operands (backends/triton/quantization.py:293-409) and the probe-matched
product (backends/triton/api.py:23-83).
"""

from __future__ import annotations

import sys

import numpy as np
import torch


def main(cases_path: str, results_path: str) -> None:
    from ue5m3_fp4.backends.triton import fake_quantize_gemm_operands, probe_matched_fp4_gemm

    import ue5m3_fp4

    assert "_ref" in ue5m3_fp4.__file__, f"not the reference package: {ue5m3_fp4.__file__}"
    cases = np.load(cases_path)
    names = sorted({key.split(".")[0] for key in cases.files})
    results = {}
    for name in names:
        block, two_d, target_a, target_b, sr_a = (float(v) for v in cases[f"{name}.meta"])
        dtype = torch.float32 if f"{name}.fp32" in cases.files else torch.bfloat16
        a = torch.from_numpy(cases[f"{name}.a"]).to(dtype).cuda()
        b = torch.from_numpy(cases[f"{name}.b"]).to(dtype).cuda()
        kwargs = dict(block_size=int(block), scale_target_a=target_a, scale_target_b=target_b,
                      two_dimensional_b=bool(two_d))
        if sr_a:
            kwargs["rounding_a"] = "StochasticFast"
            kwargs["random_bits_a"] = torch.from_numpy(cases[f"{name}.bits_a"]).to(torch.int32).cuda()
        if f"{name}.amax_a" in cases.files:
            kwargs["tensor_amax_a"] = float(cases[f"{name}.amax_a"])
        if f"{name}.amax_b" in cases.files:
            kwargs["tensor_amax_b"] = float(cases[f"{name}.amax_b"])
        for domain in ("encoded", "decoded"):
            qa, qb = fake_quantize_gemm_operands(a, b, output_domain=domain, output_dtype=torch.float32, **kwargs)
            results[f"{name}.{domain}_a"] = qa.cpu().numpy()
            results[f"{name}.{domain}_b"] = qb.cpu().numpy()
        results[f"{name}.product"] = probe_matched_fp4_gemm(a, b, **kwargs).cpu().numpy()
        torch.cuda.synchronize()
        print("reference case done:", name, flush=True)
    np.savez(results_path, **results)


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
