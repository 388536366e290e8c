"""Benchmark of the probe-matched FP4 GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one forward pass of the hot path over one batch of seeded synthetic input at
the Nemotron-H-8B MLP up-projection shape (X bf16 8192x4096 per rank, W bf16 21504x4096):
(tensor amax of X + MAX all-reduce over the data-parallel ranks on refresh steps, every
50th step as in the D=50 recipe) -> quantize X (1x16 blocks) -> quantize W (16x16 tiles)
-> issue-RZ GEMM with fused snap/alpha/bf16 epilogue.  Rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "ue5m3-fp4_b200"))

M, K, N = 8192, 4096, 21504
BLOCK = 16
TARGET = 448.0
REFRESH_INTERVAL = 50
METRIC = "probe_matched_fp4_gemm_tflops_m8192_k4096_n21504"
UNIT = "TFLOP/s"
WORKLOAD = "forward probe-matched GEMM Y=X.W^T, X bf16 8192x4096 N(0,1), W bf16 21504x4096 N(0,0.02^2), B=16"


def _peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        data["source"] = "measured"
        return data
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def _config(n_gpus: int) -> dict:
    return {
        "workload": WORKLOAD,
        "m_per_rank": M, "k": K, "n": N, "block_size": BLOCK, "scale_target": TARGET,
        "rounding": "ties_to_even", "weights": "2-D 16x16 tiles", "snap": "1/1024", "out_dtype": "bf16",
        "parallelism": f"dp{n_gpus}", "amax_refresh_every_steps": REFRESH_INTERVAL,
        "cache": "working set per step (X, W, encoded operands, Y: 0.84 GB) exceeds the 126 MB L2",
        "seed": 0,
    }


# ---------------------------------------------------------------------------------------
# clocks sampled during the timed region
# ---------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int) -> None:
        self.device_index = device_index
        self.lines: list[str] = []
        self.proc = None
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.lines.append(line.strip())

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [part.strip() for part in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, value in zip(names, parts[5:9]):
                if value.lower() == "active":
                    reasons.add(name)
        sm.sort()
        return {
            "sm_mhz": sm[len(sm) // 2] if sm else None,
            "sm_max_mhz": max(sm_max) if sm_max else None,
            "power_w_max": max(power) if power else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


# ---------------------------------------------------------------------------------------
# CPU arm: the oracle port of the same path on a bounded sample of the workload
# ---------------------------------------------------------------------------------------
def _cpu_sample_inputs(rows: int, cols: int):
    import torch

    g = torch.Generator().manual_seed(0)
    x = torch.randn(rows, K, generator=g).to(torch.bfloat16).float().numpy()
    w = (0.02 * torch.randn(cols, K, generator=g)).to(torch.bfloat16).float().numpy()
    return x, w


def _cpu_step(x, w) -> float:
    """One pass of the path on the CPU oracle; returns seconds."""

    from oracle import ue5m3_oracle as o

    start = time.perf_counter()
    o.probe_matched_fp4_gemm(x, w, block=BLOCK, target_a=TARGET, target_b=TARGET, two_dimensional_b=True, snap=True)
    return time.perf_counter() - start


def cpu_baseline(budget_s: float = 12.0) -> dict:
    from oracle import ue5m3_oracle as o

    rows, cols = 64, 256
    x, w = _cpu_sample_inputs(rows, cols)
    probe = _cpu_step(x, w)
    # grow the sample toward the budget (work scales with rows*cols)
    scale = max(1.0, min(64.0, budget_s / max(probe, 1e-3)))
    rows = int(min(M, rows * max(1, int(scale ** 0.5))))
    cols = int(min(N, cols * max(1, int(scale ** 0.5))))
    x, w = _cpu_sample_inputs(rows, cols)
    seconds = _cpu_step(x, w)
    return {
        "value": 2.0 * rows * cols * K / seconds / 1e12,
        "unit": UNIT,
        "cores": o.num_threads(),
        "kind": "port",
        "sample": f"{rows} rows of X x {cols} rows of W x K={K}: quantize both operands + exact K=64 "
                  f"issue-RZ GEMM + snap + alpha in the C oracle, {seconds:.2f} s",
    }


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ue5m3_oracle as o

    rows, cols = 256, 1024
    x, w = _cpu_sample_inputs(rows, cols)
    for _ in range(args.warmup):
        _cpu_step(x, w)
    times = [_cpu_step(x, w) for _ in range(args.steps)]
    seconds = sum(times) / len(times)
    value = 2.0 * rows * cols * K / seconds / 1e12
    sample = f"per step: {rows} rows of X x {cols} rows of W x K={K} of the workload, C oracle port, OpenMP"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp4(e2m1)xue5m3 -> fp32", "data": "synthetic",
        "config": _config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": o.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))
