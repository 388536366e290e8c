"""Benchmark of the probe-matched FP4 GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one forward pass of the hot path over one batch of seeded synthetic input at
the Nemotron-H-8B MLP up-projection shape (X bf16 8192x4096 per rank, W bf16 21504x4096):
(tensor amax of X + MAX all-reduce over the data-parallel ranks on refresh steps, every
50th step as in the D=50 recipe) -> quantize X (1x16 blocks, packed codes + scale atoms)
-> quantize W (16x16 tiles) -> FP4 block-scaled tensor-core GEMM with fused snap / alpha /
bf16 epilogue -> the device-driven recomputation pass for block scales outside the tensor
core's scale window (returns at once on this data).  Rank 0 prints one JSON line whose
`value` is that step; the same line carries the other configurations of the workload
(quantize headline and round trip, the full linear at two shapes, the Nemotron-H-shaped
data-parallel training step) as separate objects.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from contextlib import nullcontext
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "ue5m3-fp4_b200"))

M, K, N = 8192, 4096, 21504
BLOCK = 16
TARGET = 448.0
REFRESH_INTERVAL = 50
BUCKET_MB = int(os.environ.get("UE5M3_BENCH_BUCKET_MB", "200"))   # DDP gradient bucket size of the c5 leg
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
    """SM clock, power and throttle reasons polled through NVML every few milliseconds.

    The timed region of the default run lasts tens of milliseconds, shorter than one
    `nvidia-smi -lms` period, so the poll runs in-process.  `mark()` brackets the timed
    region; the summary reports the samples inside the marks (all samples when there are
    too few inside).
    """

    REASONS = {
        "hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
        "sw_power_cap": 0x4,
    }

    def __init__(self, device_index: int, period_s: float = 0.002) -> None:
        self.device_index = device_index
        self.period_s = period_s
        self.samples: list[tuple[float, int, float, int]] = []
        self.marks: list[float] = []
        self.handle = None
        self.nvml = None
        self.sm_max = None
        self.thread = None
        self.stop_flag = threading.Event()

    def _handle(self):
        import pynvml
        import torch

        pynvml.nvmlInit()
        self.nvml = pynvml
        try:
            uuid = str(torch.cuda.get_device_properties(self.device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            return pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            return pynvml.nvmlDeviceGetHandleByIndex(self.device_index)

    def start(self) -> None:
        try:
            self.handle = self._handle()
            self.sm_max = self.nvml.nvmlDeviceGetMaxClockInfo(self.handle, self.nvml.NVML_CLOCK_SM)
        except Exception:
            self.handle = None
            return

        def poll():
            nv, h = self.nvml, self.handle
            reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                nv.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self.stop_flag.is_set():
                try:
                    self.samples.append((time.perf_counter(),
                                         nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM),
                                         nv.nvmlDeviceGetPowerUsage(h) / 1000.0,
                                         int(reasons_fn(h))))
                except Exception:
                    pass
                time.sleep(self.period_s)

        self.thread = threading.Thread(target=poll, daemon=True)
        self.thread.start()

    def mark(self) -> None:
        self.marks.append(time.perf_counter())

    def stop(self) -> None:
        if self.handle is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)

    def summary(self, begin: float | None = None, end: float | None = None) -> dict:
        """Samples between two time.perf_counter() stamps (default: the first two marks); all
        samples when fewer than three fall inside."""

        if self.handle is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["NVML unavailable"]}
        rows = list(self.samples)
        window = "warm-up + timed region"
        if begin is None and len(self.marks) >= 2:
            begin, end = self.marks[0], self.marks[1]
        if begin is not None:
            inside = [r for r in rows if begin <= r[0] <= end]
            if len(inside) >= 3:
                rows, window = inside, "timed region"
        sm = sorted(r[1] for r in rows)
        bits = 0
        for r in rows:
            bits |= r[3]
        return {
            "sm_mhz": float(sm[len(sm) // 2]) if sm else None,
            "sm_min_mhz": float(sm[0]) if sm else None,
            "sm_max_mhz": float(self.sm_max) if self.sm_max else None,
            "power_w_max": max((r[2] for r in rows), default=None),
            "samples": len(sm),
            "window": window,
            "reasons": sorted(name for name, bit in self.REASONS.items() if bits & bit),
        }


# ---------------------------------------------------------------------------------------
# CPU arm: the reference's PORTABLE composition of the same path (nn/linear.py:117-218 of the
# reference: fake-quantize both operands with the formats.py block quantizer, multiply in FP32),
# restated as the C oracle's block quantizer (all host threads) + torch.mm in FP32, on the whole
# workload.  The exact-partial round-toward-zero GEMM of the oracle is a checker, not a baseline.
# ---------------------------------------------------------------------------------------
def _cpu_inputs():
    import torch

    g = torch.Generator().manual_seed(0)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).float().numpy()
    w = (0.02 * torch.randn(N, K, generator=g)).to(torch.bfloat16).float().numpy()
    return x, w


def _cpu_step(x, w) -> tuple[float, float]:
    """One pass of the portable composition on the host; returns (seconds, quantizer seconds)."""

    import torch

    from oracle import ue5m3_oracle as o

    start = time.perf_counter()
    qx = o.quantize(x, block=BLOCK, blocking=o.BLOCK_ROW, amax_value=o.amax(x), target=TARGET)["dequant"]
    qw = o.quantize(w, block=BLOCK, blocking=o.BLOCK_2D, amax_value=o.amax(w), target=TARGET)["dequant"]
    middle = time.perf_counter()
    y = torch.mm(torch.from_numpy(qx), torch.from_numpy(qw).t()).to(torch.bfloat16)
    assert y.shape == (M, N)
    end = time.perf_counter()
    return end - start, middle - start


def _cpu_threads() -> int:
    import torch

    from oracle import ue5m3_oracle as o

    cores = os.cpu_count() or 1
    o.set_threads(cores)  # launchers may have exported OMP_NUM_THREADS=1
    torch.set_num_threads(cores)
    return cores


def cpu_baseline() -> dict:
    cores = _cpu_threads()
    x, w = _cpu_inputs()
    seconds, quantize_seconds = _cpu_step(x, w)
    return {
        "value": 2.0 * M * N * K / seconds / 1e12,
        "unit": UNIT,
        "cores": cores,
        "kind": "port",
        "sample": f"the whole workload once: block-quantize X {M}x{K} and W {N}x{K} (C restatement of formats.py, "
                  f"{quantize_seconds:.2f} s) + fp32 torch.mm + bf16 cast, {seconds:.2f} s in all",
    }


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = _cpu_threads()
    x, w = _cpu_inputs()
    for _ in range(min(args.warmup, 1)):
        _cpu_step(x, w)
    steps = max(1, min(args.steps, 5))  # whole workload per step; bounded so that the run stays within minutes
    times = [_cpu_step(x, w)[0] for _ in range(steps)]
    seconds = sum(times) / len(times)
    value = 2.0 * M * N * K / seconds / 1e12
    sample = (f"per step the whole workload: block-quantize both operands (C restatement of formats.py) + fp32 torch.mm + "
              f"bf16 cast on {cores} host threads; {steps} timed steps of the {args.steps} requested")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp4 (e2m1 x ue5m3) fake-quantized, fp32 multiply", "data": "synthetic",
        "config": _config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------
class HotPath:
    """Device-resident state of one rank and the launches of one step."""

    def __init__(self, device, rank: int, world: int) -> None:
        import torch
        from ue5m3_fp4.backends import b200

        self.torch, self.ops, self.device, self.world = torch, b200, device, world
        g = torch.Generator().manual_seed(1000 + rank)  # each data-parallel rank has its own batch
        gw = torch.Generator().manual_seed(0)  # weights are replicated
        self.x_host = torch.randn(M, K, generator=g).to(torch.bfloat16).pin_memory()
        self.x = self.x_host.to(device)
        self.w = (0.02 * torch.randn(N, K, generator=gw)).to(torch.bfloat16).to(device)
        # end-to-end leg: two input slots on the device, two pinned result buffers, one stream
        # per copy direction, so that step i+1's input and step i-1's result move while step i runs
        self.y_host = [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        self.x_slots = [self.x, torch.empty_like(self.x)]
        self.copy_in, self.copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self.x_ready = [torch.cuda.Event() for _ in range(2)]
        self.x_free = [torch.cuda.Event() for _ in range(2)]
        self.e2e_index = 0
        self.amax_w = b200.tensor_amax(self.w).reshape(1)  # held: sampled once at "step 1"
        self.amax_x = b200.tensor_amax(self.x).reshape(1)
        self.gemm_events: list = []
        self.step_index = 0
        self.path = b200.gemm_path()

    def refresh_activation_amax(self, x) -> None:
        """Sample max|X| on the device and MAX all-reduce it across the data-parallel ranks."""

        torch = self.torch
        self.amax_x = self.ops.tensor_amax(x).reshape(1)
        if self.world > 1:
            torch.distributed.all_reduce(self.amax_x, op=torch.distributed.ReduceOp.MAX)

    def step(self, time_gemm: bool = False, x=None):
        torch, ops = self.torch, self.ops
        x = self.x if x is None else x
        if self.step_index % REFRESH_INTERVAL == 0:
            self.refresh_activation_amax(x)
        self.step_index += 1
        alpha = ops.EpilogueAlpha.of(self.amax_x, self.amax_w, TARGET, TARGET)  # formed in the GEMM epilogue
        if self.path == "fp4":
            # packed codes + scale bytes, scales re-laid for the tensor core, FP4 MMA
            xq = ops.quantize_fp4_operand(x, block_size=BLOCK, blocking=ops.BLOCK_ROW, transposed=False,
                                          tensor_amax=self.amax_x, scale_target=TARGET)
            wq = ops.quantize_fp4_operand(self.w, block_size=BLOCK, blocking=ops.BLOCK_2D, transposed=False,
                                          tensor_amax=self.amax_w, scale_target=TARGET)
        else:
            xq = ops.quantize_packed(x, block_size=BLOCK, blocking=ops.BLOCK_ROW, tensor_amax=self.amax_x,
                                     scale_target=TARGET, packed=False, fake_domain="encoded",
                                     fake_dtype=torch.bfloat16).fake
            wq = ops.quantize_packed(self.w, block_size=BLOCK, blocking=ops.BLOCK_2D, tensor_amax=self.amax_w,
                                     scale_target=TARGET, packed=False, packed_t=False, fake_domain="encoded",
                                     fake_dtype=torch.bfloat16).fake
        events = None
        if time_gemm:
            events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self.gemm_events.append(events)
        if self.path == "fp4":
            # the events bracket the FP4 GEMM launch alone: the placement before it and the
            # recomputation pass after it are separate kernels of the step
            y = ops.gemm_fp4_operands(xq, wq, snap=True, alpha=alpha, out_dtype=torch.bfloat16, kernel_events=events)
        else:
            if events:
                events[0].record()
            y = ops.gemm_issue_rz(xq, wq, snap=True, alpha=alpha, out_dtype=torch.bfloat16)
            if events:
                events[1].record()
        return y

    def step_e2e(self):
        """The same step behind host buffers: X from pinned host memory in, Y to pinned host
        memory out, every step; the two copy directions run on their own streams and overlap
        the neighbouring steps' compute."""

        torch = self.torch
        slot = self.e2e_index % 2
        self.e2e_index += 1
        main = torch.cuda.current_stream()
        self.copy_in.wait_event(self.x_free[slot])  # the step that last read this slot has finished
        with torch.cuda.stream(self.copy_in):
            self.x_slots[slot].copy_(self.x_host, non_blocking=True)
            self.x_ready[slot].record(self.copy_in)
        main.wait_event(self.x_ready[slot])
        y = self.step(x=self.x_slots[slot])
        self.x_free[slot].record(main)
        self.copy_out.wait_stream(main)
        with torch.cuda.stream(self.copy_out):
            self.y_host[slot].copy_(y, non_blocking=True)  # same stream as the copy two steps ago
        y.record_stream(self.copy_out)
        return y

    def finish_e2e(self) -> None:
        """Make the timing stream wait for the last result copy."""

        self.torch.cuda.current_stream().wait_stream(self.copy_out)


def _timed(torch, dist, world, fn, steps: int, finish=None) -> float:
    """Seconds for `steps` calls of fn: barrier + synchronize on both sides, CUDA events, max over ranks.
    `finish` joins side streams into the timing stream before the closing event."""

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    if finish is not None:
        finish()
    stop.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    elapsed = torch.tensor([start.elapsed_time(stop) / 1e3], device="cuda")
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    return float(elapsed.item())


def _quantize_headline(torch, ops, device, steps: int, peaks: dict) -> dict:
    """Backward-operand quantize of dY: bf16 8192x4096, Student-t(3)*1e-3, B=16 1-D blocks,
    StochasticFast with a seeded uint8 bit tensor, held amax; packed nibbles + scale bytes out.

    Kernel-only timing through the C ABI with preallocated outputs: `steps` back-to-back
    launches between two CUDA events, rotating over four distinct input sets (4 x 100 MB,
    larger than the 126 MB L2) so that every launch reads from HBM."""

    from ue5m3_fp4 import _native

    lib = _native.load()
    sets = []
    for seed in range(4):
        g = torch.Generator().manual_seed(seed)
        z = torch.randn(M, K, generator=g)
        chi = torch.randn(3, M, K, generator=g).square().sum(0)
        dy = (z / torch.sqrt(chi / 3.0) * 1e-3).to(torch.bfloat16).to(device)
        bits = torch.randint(0, 256, (M, K), generator=g, dtype=torch.int32).to(torch.uint8).to(device)
        sets.append((dy, bits))
    amax = ops.tensor_amax(sets[0][0]).reshape(1)
    codes = torch.empty((M, K // 2), dtype=torch.uint8, device=device)
    scales = torch.empty((M, K // BLOCK), dtype=torch.uint8, device=device)
    stream = _native.stream_ptr(device)

    def launch(i: int, sr: bool) -> None:
        dy, bits = sets[i % 4]
        status = lib.ue5m3_quantize(
            dy.data_ptr(), _native.DTYPE_BF16, M, K, BLOCK, _native.BLOCK_ROW, amax.data_ptr(), TARGET,
            _native.ROUND_STOCHASTIC_FAST if sr else _native.ROUND_TIES_TO_EVEN,
            bits.data_ptr() if sr else None, _native.BITS_U8 if sr else _native.BITS_NONE,
            codes.data_ptr(), scales.data_ptr(), None, None, None, None, 0, 0, stream)
        _native.check(status, "ue5m3_quantize")

    def run(sr: bool) -> float:
        for i in range(4):
            launch(i, sr)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            launch(i, sr)
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) * 1e-3 / steps

    elems = M * K
    sr_s, tte_s = run(True), run(False)
    sr_bytes = elems * (2 + 1 + 0.5 + 1.0 / BLOCK)
    tte_bytes = elems * (2 + 0.5 + 1.0 / BLOCK)
    return {
        "workload": "dY bf16 8192x4096 Student-t(3)*1e-3, B=16, held amax; four rotating input sets (> L2)",
        "launches_timed": steps,
        "stochastic_u8_bits": {"us": sr_s * 1e6, "achieved_gbs": sr_bytes / sr_s / 1e9,
                               "frac_of_hbm_peak": sr_bytes / sr_s / 1e9 / peaks["hbm_gbs"],
                               "algorithmic_bytes": sr_bytes},
        "ties_to_even": {"us": tte_s * 1e6, "achieved_gbs": tte_bytes / tte_s / 1e9,
                         "frac_of_hbm_peak": tte_bytes / tte_s / 1e9 / peaks["hbm_gbs"],
                         "algorithmic_bytes": tte_bytes},
        "peak_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"],
    }


def _library_fp4_reference(torch, device):
    """cuBLASLt's NVFP4 GEMM (torch._scaled_mm, block-16 UE4M3 scales) on the benchmark shape,
    random codes: a measured library figure beside the roofline (the measured-peaks file has no FP4
    entry).  Runs after the timed regions; returns TFLOP/s or None when the build lacks the path."""

    try:
        a = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, device=device).view(torch.float4_e2m1fn_x2)
        b = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=device).view(torch.float4_e2m1fn_x2)
        pad = lambda rows: (rows + 127) // 128 * 128 * ((K // 16 + 3) // 4 * 4)
        sa = torch.full((pad(M),), 0.5, device=device).to(torch.float8_e4m3fn)
        sb = torch.full((pad(N),), 0.5, device=device).to(torch.float8_e4m3fn)
        run = lambda: torch._scaled_mm(a, b.t(), sa, sb, out_dtype=torch.bfloat16)
        for _ in range(3):
            run()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(20):
            run()
        stop.record()
        torch.cuda.synchronize(device)
        return 2.0 * M * N * K / (start.elapsed_time(stop) / 20 * 1e-3) / 1e12
    except Exception:  # noqa: BLE001 - optional reference, any failure just omits it
        return None


def _linear_case(torch, device, *, tokens: int, in_f: int, out_f: int, block: int, name: str, activation: str,
                 dy_scale: float, steps: int, what: str) -> dict:
    """Forward + backward of one UE5M3Linear (three GEMMs, their operand quantizations, the amax
    lifecycle at a hold step), CUDA events around `steps` repetitions on resident inputs."""

    from ue5m3_fp4.nn import UE5M3Linear
    from ue5m3_fp4.recipe import UE5M3Recipe

    try:
        recipe = UE5M3Recipe.proposed()
        if block != 16:
            recipe = UE5M3Recipe.from_dict({**recipe.to_dict(), "block_size": block, "name": f"b{block}"})
        layer = UE5M3Linear(in_f, out_f, bias=False, recipe=recipe, backend="probe_matched", module_name=name,
                            device=device, dtype=torch.bfloat16)
        g = torch.Generator(device=device).manual_seed(3)
        with torch.no_grad():
            layer.weight.copy_(0.02 * torch.randn(out_f, in_f, device=device, generator=g))
        z = torch.randn(tokens, in_f, device=device, generator=g)
        x = (torch.relu(z).square_() if activation == "squared_relu" else z).to(torch.bfloat16).requires_grad_(True)
        del z
        dy = (dy_scale * torch.randn(tokens, out_f, device=device, generator=g)).to(torch.bfloat16)
        layer.scale_state.begin_step(1)

        def one():
            layer.weight.grad = None
            x.grad = None
            layer(x).backward(dy)

        for _ in range(3):
            one()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            one()
        stop.record()
        torch.cuda.synchronize(device)
        ms = start.elapsed_time(stop) / steps
        # rows / columns that the recomputation pass took over (block scales outside the UE4M3 window)
        from ue5m3_fp4.backends import b200
        from ue5m3_fp4.nn import linear as linear_module

        plan = linear_module._OperandPlan(layer)
        reference = layer.scale_state.reference("activation", name, x.detach())
        fwd = b200.quantize_fp4_operand(x.detach(), block_size=block, blocking=b200.BLOCK_ROW, transposed=False,
                                        tensor_amax=reference.reshape(1), scale_target=plan.target("activation"),
                                        shift_headroom=1)
        wgrad = b200.quantize_fp4_operand(x.detach(), block_size=block, blocking=b200.BLOCK_COL, transposed=True,
                                          tensor_amax=reference.reshape(1), scale_target=plan.target("activation"),
                                          shift_headroom=1)
        return {"what": what, "ms": ms, "tflops": 3 * 2.0 * tokens * in_f * out_f / (ms * 1e-3) / 1e12, "steps": steps,
                "fallback_rows": {"forward_x_rows": fwd.window_counts()[0], "wgrad_x_columns": wgrad.window_counts()[0]}}
    except Exception as error:  # noqa: BLE001 - informational leg
        return {"what": what, "error": f"{type(error).__name__}: {error}"[:300]}


def _round_trip_c1(torch, ops, device, steps: int, peaks: dict) -> dict:
    """fp32 4096 x 4096, N(0,1) with 1 % of the entries x 100, B = 16, target 448 from the current
    tensor's amax (D = 1), ties to even: amax pass + packed codes + scale bytes + dequantized fp32.
    Rotates over three input sets (3 x 67 MB inputs and 3 x 67 MB outputs, beyond L2)."""

    rows = cols = 4096
    sets = []
    for seed in range(3):
        g = torch.Generator(device=device).manual_seed(seed)
        x = torch.randn(rows, cols, device=device, generator=g)
        sets.append(torch.where(torch.rand(rows, cols, device=device, generator=g) < 0.01, x * 100.0, x))

    def one(i: int):
        x = sets[i % 3]
        amax = ops.tensor_amax(x).reshape(1)
        return ops.quantize_packed(x, block_size=16, tensor_amax=amax, scale_target=TARGET, rounding="TTE",
                                   fake_domain="dequant", fake_dtype=torch.float32)

    for i in range(3):
        one(i)
    torch.cuda.synchronize(device)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        one(i)
    stop.record()
    torch.cuda.synchronize(device)
    seconds = start.elapsed_time(stop) * 1e-3 / steps
    algorithmic = rows * cols * (4 + 4 + 0.5 + 1.0 / 16 + 4)
    return {"workload": "fp32 4096x4096, N(0,1) with 1% x100 outliers, B=16, current-tensor amax, TTE: amax pass + codes + "
                        "scale bytes + dequantized fp32 (two launches per round trip)",
            "us": seconds * 1e6, "algorithmic_bytes": algorithmic, "achieved_gbs": algorithmic / seconds / 1e9,
            "frac_of_hbm_peak": algorithmic / seconds / 1e9 / peaks["hbm_gbs"], "launches_timed": 2 * steps}


def _c5_training_step(torch, dist, device, rank: int, world: int, local_rank: int, compare_bf16: bool = True) -> dict:
    """One data-parallel training step of the Nemotron-H-8B-shaped stack (112 FP4 linears at their
    real shapes, stand-in mixers, FP32 vocabulary head): uniform random token ids, sequence 8192,
    micro-batch 1 per GPU, forward + backward + optimizer step, torch DDP with bf16 gradient
    buckets reduced during the backward pass, amax MAX all-reduces on refresh steps."""

    import torch.nn.functional as F
    from torch.nn.parallel import DistributedDataParallel

    from ue5m3_fp4.integrations.torchtitan.selection import convert_reported_nemotron_h
    from ue5m3_fp4.integrations.torchtitan.shaped_stack import NemotronHShapedStack
    from ue5m3_fp4.integrations.torchtitan.trainer import begin_training_step

    seq = 8192
    try:
        torch.manual_seed(0)  # replicated weights
        model = NemotronHShapedStack(device=device, dtype=torch.bfloat16)
        model.lm_head.to(torch.float32)  # the vocabulary head keeps FP32 parameters
        conversion = convert_reported_nemotron_h(model)
        from ue5m3_fp4.nn import reserve_device_workspace

        reserve_device_workspace(conversion.fp4_linears, seq, device)   # no step grows the recomputation workspace
        previous_tf32 = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True  # stated policy of the stand-in's FP32 head: TF32 tensor cores
        parameters = sum(p.numel() for p in model.parameters())
        gradient_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
        wrapped = model
        if world > 1:
            wrapped = DistributedDataParallel(model, device_ids=[local_rank], gradient_as_bucket_view=True,
                                              bucket_cap_mb=BUCKET_MB, broadcast_buffers=False)
        # learning rate 0: the optimizer step runs in full (same kernels, same memory traffic) but the
        # weights keep the statistics of their random initialisation, so that the synthetic
        # activations and gradients do not drift toward whatever a repeated random batch rewards
        optimizer = torch.optim.AdamW(model.parameters(), lr=0.0, fused=True)
        g = torch.Generator(device=device).manual_seed(100 + rank)

        def step(index: int, sync: bool = True) -> None:
            ids = torch.randint(0, model.config.vocab_size, (1, seq), device=device, generator=g)  # fresh batch
            labels = torch.roll(ids, -1, dims=1).reshape(-1)
            begin_training_step([model], index)
            context = nullcontext() if (sync or world == 1) else wrapped.no_sync()
            with context:
                logits = wrapped(ids)
                loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]), labels)
                loss.backward()
            optimizer.step()   # also in the run without gradient all-reduce, so that the two differ by it alone
            optimizer.zero_grad(set_to_none=True)

        def timed(indices, sync: bool = True) -> float:
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize(device)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for index in indices:
                step(index, sync)
            stop.record()
            torch.cuda.synchronize(device)
            elapsed = torch.tensor([start.elapsed_time(stop) / len(indices)], device=device)
            if world > 1:
                dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
            return float(elapsed.item())

        step(1)   # first refresh step: also absorbs one-time library initialisation
        step(2)
        step(3)   # the caching allocator has seen every size of a step by now
        hold_ms = timed([4, 5, 6, 7, 8])
        local_ms = timed([9, 10, 11], sync=False) if world > 1 else None   # same step without gradient all-reduce
        refresh_ms = (timed([60]) + timed([110])) / 2   # every reference is due again: 336 amax samples
        entries = conversion.scale_state.report()["entries"]
        conversion.scale_state.verify_samples()
        from ue5m3_fp4.backends import b200

        b200.log_window_records(True)   # one more step, untimed: how much of it the recomputation pass took over
        step(111)
        torch.cuda.synchronize(device)
        window = b200.window_log_summary()
        b200.log_window_records(False)
        b200.check_gemm_status(device)
        peak_memory = torch.cuda.max_memory_allocated(device)
        torch.backends.cuda.matmul.allow_tf32 = previous_tf32
        result = {
            "what": "Nemotron-H-8B-shaped stack (52 layers, 112 FP4 linears B=16 at their real shapes, stand-in mixers, "
                    "FP32 head with TF32 matmul), uniform random token ids drawn per step, seq 8192, micro-batch 1 per GPU, "
                    "forward + backward + fused AdamW (bf16 parameters and optimizer state, learning rate 0), torch DDP, "
                    f"bf16 gradient buckets of {BUCKET_MB} MB",
            "tokens_per_s": seq * world / (hold_ms * 1e-3), "ms_hold_step": hold_ms, "ms_refresh_step": refresh_ms,
            "tokens_per_s_refresh_step": seq * world / (refresh_ms * 1e-3),
            "ms_hold_step_without_gradient_allreduce": local_ms,
            "exposed_gradient_allreduce_ms": None if local_ms is None else hold_ms - local_ms,
            "gradient_bytes_reduced_per_rank_step": gradient_bytes if world > 1 else 0,
            "amax_entries": len(entries), "amax_collectives_refresh_step": (1 + 224) if world > 1 else 0,
            "amax_collectives_hold_step": 0,
            "fp4_linear_tflops_per_rank": model.fp4_linear_flops_per_token() * seq / (hold_ms * 1e-3) / 1e12,
            "parameters": parameters, "peak_memory_gb": peak_memory / 1e9, "n_gpus": world,
            "scale_window": window,
        }
        del optimizer, wrapped, model
        torch.cuda.empty_cache()
        if world == 1 and compare_bf16:
            # the same stack and step with its 112 linears left as bf16 nn.Linear (cuBLAS): what the
            # FP4 path costs or saves at the level of a training step
            result["ms_hold_step_bf16_linears"] = _c5_bf16_step(torch, device, seq)
        return result
    except Exception as error:  # noqa: BLE001 - reported, the headline does not depend on it
        import traceback

        return {"error": f"{type(error).__name__}: {error}"[:400], "trace": traceback.format_exc()[-600:]}


def _c5_bf16_step(torch, device, seq: int) -> float | str:
    """ms per step of the unconverted Nemotron-H-shaped stack (bf16 linears), same batch, optimizer and head."""

    import torch.nn.functional as F

    from ue5m3_fp4.integrations.torchtitan.shaped_stack import NemotronHShapedStack

    try:
        torch.manual_seed(0)
        model = NemotronHShapedStack(device=device, dtype=torch.bfloat16)
        model.lm_head.to(torch.float32)   # FP32 head on FP32 inputs, as the converted stack has it
        model.lm_head.register_forward_pre_hook(lambda module, inputs: (inputs[0].float(),))
        previous_tf32 = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        optimizer = torch.optim.AdamW(model.parameters(), lr=0.0, fused=True)
        g = torch.Generator(device=device).manual_seed(100)

        def step() -> None:
            ids = torch.randint(0, model.config.vocab_size, (1, seq), device=device, generator=g)
            labels = torch.roll(ids, -1, dims=1).reshape(-1)
            logits = model(ids)
            F.cross_entropy(logits.reshape(-1, logits.shape[-1]), labels).backward()
            optimizer.step()
            optimizer.zero_grad(set_to_none=True)

        step()
        step()
        torch.cuda.synchronize(device)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(3):
            step()
        stop.record()
        torch.cuda.synchronize(device)
        torch.backends.cuda.matmul.allow_tf32 = previous_tf32
        elapsed = start.elapsed_time(stop) / 3
        del optimizer, model
        torch.cuda.empty_cache()
        return elapsed
    except Exception as error:  # noqa: BLE001 - a comparison figure only
        return f"{type(error).__name__}: {error}"[:300]


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from ue5m3_fp4.backends import b200

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path for the product arm")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    if not b200.available():
        raise SystemExit("the sm_100a library is not built: run python ue5m3-fp4_b200/build.py")
    peaks = _peaks()
    hot = HotPath(device, rank, world)
    # UE5M3_BENCH_LEGS=c5,linear ... restricts the side legs while developing; the default runs all
    chosen = {leg.strip() for leg in os.environ.get("UE5M3_BENCH_LEGS", "all").split(",")}
    leg = lambda name: "all" in chosen or name in chosen  # noqa: E731

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # samples cover warm-up (same work) and the timed regions
    for _ in range(max(args.warmup, 3)):
        hot.step()
    from ue5m3_fp4 import _native

    launches_before = _native.launch_count
    hot.step_index = 0
    sampler.mark()
    seconds = _timed(torch, dist, world, lambda: hot.step(time_gemm=True), args.steps)
    sampler.mark()
    launches = _native.launch_count - launches_before  # kernels of the library inside the timed region
    b200.check_gemm_status(device)
    gemm_s = sum(a.elapsed_time(b) for a, b in hot.gemm_events) / len(hot.gemm_events) / 1e3

    # sustained leg: the same step back to back for at least two seconds (the regime of a training run)
    sustained_steps = max(args.steps, int(2.2 / max(seconds / args.steps, 1e-5)))
    hot.gemm_events.clear()
    sustained_begin = time.perf_counter()
    sustained_seconds = _timed(torch, dist, world, lambda: hot.step(time_gemm=True), sustained_steps)
    sustained_end = time.perf_counter()
    tail = hot.gemm_events[len(hot.gemm_events) // 2:]  # second half: clocks have settled
    gemm_sustained_s = sum(a.elapsed_time(b) for a, b in tail) / len(tail) / 1e3
    hot.gemm_events.clear()

    for _ in range(2):
        hot.step_e2e()
    e2e_seconds = _timed(torch, dist, world, hot.step_e2e, args.steps, finish=hot.finish_e2e)
    sampler.stop()

    flops_per_rank = 2.0 * M * N * K
    value = flops_per_rank * world * args.steps / seconds / 1e12
    e2e_value = flops_per_rank * world * args.steps / e2e_seconds / 1e12
    fp4 = hot.path == "fp4"
    line = None
    if rank == 0:
        clocks = sampler.summary()
        sustained_clocks = sampler.summary(sustained_begin, sustained_end)
        quant = _quantize_headline(torch, b200, device, max(args.steps, 40), peaks) if leg("quantize") else {}
        if leg("quantize"):
            quant["c1_round_trip"] = _round_trip_c1(torch, b200, device, 30, peaks)
        cpu = cpu_baseline() if world == 1 and leg("cpu") else None
        # The FP4 kernel issues kind::mxf4nvf4 MMAs, four times the BF16 MMA rate of the same tensor
        # core; no FP4 peak is measured, so the denominators are 4 x the measured cuBLAS BF16
        # figures: the burst one for the in-step CUDA-event time of the short run, the sustained
        # one for the two-second loop.  The nominal dense FP4 figure is 9000 TFLOP/s.
        scale = 4.0 if fp4 else 1.0
        peak_burst, peak_sustained = scale * peaks["bf16_tflops"], scale * peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
        achieved = flops_per_rank / gemm_s / 1e12
        achieved_sustained = flops_per_rank / gemm_sustained_s / 1e12
        gemm_kernel = ("gemm_fp4_pair_kernel" if os.environ.get("UE5M3_FP4_CTA_PAIR", "1") != "0" else "gemm_fp4_kernel") \
            if fp4 else "gemm_issue_rz_kernel"
        library_tf = _library_fp4_reference(torch, device) if fp4 and leg("library") else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": seconds / args.steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": ("fp4 (e2m1 x ue5m3->ue4m3 block scales) tensor-core MMA, fp32 accumulate" if fp4
                      else "fp4(e2m1)xue5m3 codes as encoded bf16 -> fp32 RZ accumulate"),
            "data": "synthetic", "config": _config(world),
            "roofline": {
                "kernel": gemm_kernel, "bound": "tensor",
                "achieved": achieved, "peak": peak_burst, "unit": "TFLOP/s", "frac": achieved / peak_burst,
                # DRAM bytes per launch: ncu capture of the M4096 N8192 case (reads 1.03 x the operand
                # bytes) scaled by the operand bytes of this shape, plus the bf16 output once
                "traffic": (1.03 * (M * K / 2 + N * K / 2 + (M + N) * K / 16) + M * N * 2) if fp4 else None,
                "peak_source": (f"4 x {peaks['source']} cuBLAS bf16 burst ({peaks['bf16_tflops']}): kernel timed with CUDA "
                                f"events inside a {seconds * 1e3:.0f} ms run" if fp4
                                else f"{peaks['source']} cuBLAS bf16 burst"),
                "frac_of_nominal_fp4_9000": achieved / 9000.0,
                "library_reference": (None if library_tf is None else {
                    "what": "cuBLASLt NVFP4 GEMM via torch._scaled_mm, same shape, random codes, 20 launches",
                    "tflops": library_tf, "frac": achieved / library_tf}),
                "algorithmic_flops_per_launch": flops_per_rank, "gemm_ms": gemm_s * 1e3,
                "sustained": {
                    "what": f"the same step back to back for {sustained_seconds:.2f} s ({sustained_steps} steps); GEMM time = "
                            "mean of the second half's CUDA-event pairs",
                    "gemm_ms": gemm_sustained_s * 1e3, "achieved": achieved_sustained, "peak": peak_sustained,
                    "frac": achieved_sustained / peak_sustained, "frac_of_nominal_fp4_9000": achieved_sustained / 9000.0,
                    "step_ms": sustained_seconds / sustained_steps * 1e3,
                    "step_tflops": flops_per_rank * world * sustained_steps / sustained_seconds / 1e12,
                    "clocks": sustained_clocks,
                    "gemm_ms_x_median_sm_mhz": (gemm_sustained_s * 1e3 * sustained_clocks["sm_mhz"]
                                                if sustained_clocks.get("sm_mhz") else None),
                    "peak_source": f"4 x {peaks['source']} cuBLAS bf16 sustained" if fp4 else f"{peaks['source']} cuBLAS bf16 sustained",
                },
            },
            "gemm_kernel": gemm_kernel,
            "quantize": quant,
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_seconds / args.steps * 1e3,
                    "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2,
                    "note": "every step: X from pinned host memory in, bf16 Y to pinned host memory out (W resident); the two "
                            "copy directions run on their own streams and overlap the neighbouring steps.  The step is bound "
                            "by the 352 MB result copy over PCIe (about 56 GB/s), not by the GPU; with N ranks on one host all "
                            "result copies share the host's PCIe root and memory bandwidth, so this figure does not scale with N "
                            "(there is no collective in it) - a linear's output normally stays on the device"},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
    # free the C3 buffers before the larger configurations
    del hot
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and leg("linear"):
        line["linear_step"] = _linear_case(
            torch, device, tokens=M, in_f=K, out_f=N, block=16, name="layers.1.mixer.up_proj", activation="normal",
            dy_scale=1e-3, steps=10, what="UE5M3Linear forward + backward, up_proj: tokens 8192, in 4096, out 21504, B=16, X ~ N(0,1)")
        line["linear_step_down_proj"] = _linear_case(
            torch, device, tokens=M, in_f=N, out_f=K, block=16, name="layers.1.mixer.down_proj", activation="squared_relu",
            dy_scale=1e-4, steps=10,
            what="UE5M3Linear forward + backward, down_proj: tokens 8192, in 21504, out 4096, B=16, X = relu(z)^2 (block scales "
                 "below the UE4M3 window occur: fallback_rows are recomputed by the BF16-issue pass)")
        torch.cuda.empty_cache()
        line["c4"] = _linear_case(
            torch, device, tokens=16384, in_f=N, out_f=K, block=32, name="layers.45.mixer.down_proj", activation="squared_relu",
            dy_scale=1e-4, steps=5,
            what="full FP4 linear forward + backward, down_proj B=32: X 16384x21504 relu(z)^2, W 4096x21504, dY 16384x4096 "
                 "N(0,1e-4^2), StochasticFast on dY, target 2048 on dY for dW, hold step of the D=50 lifecycle")
        torch.cuda.empty_cache()
    if leg("c5"):
        c5 = _c5_training_step(torch, dist, device, rank, world, local_rank)
        if rank == 0:
            line["c5"] = c5
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_case(args) -> None:
    """Small single-kernel cases for profiler captures (no JSON line, not a benchmark)."""

    import torch

    from ue5m3_fp4.backends import b200

    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(0)
    if args.case == "c5-step":
        # the Nemotron-H-shaped training step alone (launch-list captures of one step: 336 products)
        result = _c5_training_step(torch, None, device, 0, 1, 0, compare_bf16=False)
        print(json.dumps({k: result.get(k) for k in ("ms_hold_step", "ms_refresh_step", "error")}))
        return
    if args.case == "gemm-small":
        m, n = 4096, 8192  # operands + output 160 MB: larger than L2, 2048 tiles
        a = torch.randn(m, K, generator=g).to(torch.bfloat16).to(device)
        b = (0.02 * torch.randn(n, K, generator=g)).to(torch.bfloat16).to(device)
        amax_a, amax_b = b200.tensor_amax(a).reshape(1), b200.tensor_amax(b).reshape(1)
        ae = b200.quantize_packed(a, block_size=BLOCK, tensor_amax=amax_a, packed=False, fake_domain="encoded",
                                  fake_dtype=torch.bfloat16).fake
        be = b200.quantize_packed(b, block_size=BLOCK, blocking=b200.BLOCK_2D, tensor_amax=amax_b, packed=False,
                                  packed_t=False, fake_domain="encoded", fake_dtype=torch.bfloat16).fake
        alpha = b200.encoded_global_alpha(amax_a, amax_b, TARGET, TARGET)
        for _ in range(args.steps):
            b200.gemm_issue_rz(ae, be, snap=True, alpha=alpha, out_dtype=torch.bfloat16)
    elif args.case == "gemm-fp4-small":
        m, n = 4096, 8192
        a = torch.randn(m, K, generator=g).to(torch.bfloat16).to(device)
        b = (0.02 * torch.randn(n, K, generator=g)).to(torch.bfloat16).to(device)
        amax_a, amax_b = b200.tensor_amax(a).reshape(1), b200.tensor_amax(b).reshape(1)
        qa = b200.quantize_fp4_operand(a, block_size=BLOCK, blocking=b200.BLOCK_ROW, transposed=False,
                                       tensor_amax=amax_a, scale_target=TARGET)
        qb = b200.quantize_fp4_operand(b, block_size=BLOCK, blocking=b200.BLOCK_2D, transposed=False,
                                       tensor_amax=amax_b, scale_target=TARGET)
        alpha = b200.encoded_global_alpha(amax_a, amax_b, TARGET, TARGET)
        for _ in range(args.steps):
            b200.gemm_fp4_operands(qa, qb, snap=True, alpha=alpha, out_dtype=torch.bfloat16)
    elif args.case == "fallback-small":
        # squared-ReLU activations at B=16: some block scales leave the tensor core's window, so the
        # row placement and the recomputation pass have work to do (X 4096x8192, W 2048x8192)
        m, n, kk = 4096, 2048, 8192
        gd = torch.Generator(device=device).manual_seed(0)
        a = torch.relu(torch.randn(m, kk, device=device, generator=gd)).square_().to(torch.bfloat16)
        b = (0.02 * torch.randn(n, kk, device=device, generator=gd)).to(torch.bfloat16)
        amax_a, amax_b = b200.tensor_amax(a).reshape(1), b200.tensor_amax(b).reshape(1)
        alpha = b200.EpilogueAlpha.of(amax_a, amax_b, TARGET, TARGET)
        for _ in range(args.steps):
            qa = b200.quantize_fp4_operand(a, block_size=BLOCK, blocking=b200.BLOCK_ROW, transposed=False,
                                           tensor_amax=amax_a, scale_target=TARGET, shift_headroom=1)
            qb = b200.quantize_fp4_operand(b, block_size=BLOCK, blocking=b200.BLOCK_2D, transposed=False,
                                           tensor_amax=amax_b, scale_target=TARGET, shift_headroom=1)
            b200.gemm_fp4_operands(qa, qb, snap=True, alpha=alpha, out_dtype=torch.bfloat16)
        torch.cuda.synchronize()
        print("flagged rows", qa.window_counts(), "placement: listed", len(qa.placement()[0]), "placed", len(qa.placement()[1]))
    elif args.case == "linear-step":
        # forward + backward of one UE5M3Linear of the benchmark shape (launch-list captures)
        from ue5m3_fp4.nn import UE5M3Linear

        layer = UE5M3Linear(K, N, bias=False, backend="probe_matched", module_name="layers.0.mixer.up_proj",
                            device=device, dtype=torch.bfloat16)
        with torch.no_grad():
            layer.weight.copy_((0.02 * torch.randn(N, K, generator=g)).to(torch.bfloat16))
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(device).requires_grad_(True)
        dy = (1e-3 * torch.randn(M, N, generator=g)).to(torch.bfloat16).to(device)
        layer.scale_state.begin_step(1)
        for _ in range(args.steps):
            layer.weight.grad = None
            x.grad = None
            layer(x).backward(dy)
    else:
        z = torch.randn(M, K, generator=g)
        chi = torch.randn(3, M, K, generator=g).square().sum(0)
        dy = (z / torch.sqrt(chi / 3.0) * 1e-3).to(torch.bfloat16).to(device)
        bits = torch.randint(0, 256, (M, K), generator=g, dtype=torch.int32).to(torch.uint8).to(device)
        amax = b200.tensor_amax(dy).reshape(1)
        w = (0.02 * torch.randn(8192, K, generator=g)).to(torch.bfloat16).to(device)
        amax_w = b200.tensor_amax(w).reshape(1)
        for _ in range(args.steps):
            b200.quantize_packed(dy, block_size=BLOCK, tensor_amax=amax, rounding="StochasticFast", random_bits=bits)
            b200.quantize_packed(dy, block_size=BLOCK, tensor_amax=amax)
            b200.quantize_packed(dy, block_size=BLOCK, tensor_amax=amax, packed=False, fake_domain="encoded",
                                 fake_dtype=torch.bfloat16)
            b200.quantize_packed(w, block_size=BLOCK, blocking=b200.BLOCK_2D, tensor_amax=amax_w, packed=False,
                                 packed_t=False, fake_domain="encoded", fake_dtype=torch.bfloat16)
            b200.quantize_packed(dy, block_size=BLOCK, blocking=b200.BLOCK_COL, tensor_amax=amax,
                                 rounding="StochasticFast", random_bits=bits, packed=False, packed_t=False,
                                 fake_domain="encoded", fake_dtype=torch.bfloat16, fake=False, fake_t=True)
            b200.quantize_fp4_operand(dy, block_size=BLOCK, blocking=b200.BLOCK_ROW, transposed=False,
                                      tensor_amax=amax, scale_target=TARGET, rounding="StochasticFast",
                                      random_bits=bits, shift_headroom=1)
            b200.quantize_fp4_operand(w, block_size=BLOCK, blocking=b200.BLOCK_2D, transposed=False,
                                      tensor_amax=amax_w, scale_target=TARGET)
    torch.cuda.synchronize()
    b200.check_gemm_status(device)
    print("case", args.case, "done")


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--case", default=None, choices=["gemm-small", "gemm-fp4-small", "quantize", "linear-step", "fallback-small", "c5-step"],
                        help="run one small kernel case for a profiler capture instead of the benchmark")
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = parser.parse_args()
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
