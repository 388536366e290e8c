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

    def stop(self) -> dict:
        if self.handle is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["NVML unavailable"]}
        self.stop_flag.set()
        self.thread.join(timeout=2)
        rows = self.samples
        window = "warm-up + timed region"
        if len(self.marks) >= 2:
            inside = [r for r in rows if self.marks[0] <= r[0] <= self.marks[-1]]
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

    o.set_threads(os.cpu_count() or 1)  # launchers may have exported OMP_NUM_THREADS=1
    rows, cols = 64, 256
    x, w = _cpu_sample_inputs(rows, cols)
    probe = _cpu_step(x, w)
    # grow the sample toward the budget (work scales with rows*cols)
    scale = max(1.0, min(400.0, budget_s / max(probe, 1e-3)))
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

    o.set_threads(os.cpu_count() or 1)  # torchrun exports OMP_NUM_THREADS=1
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
        alpha = ops.encoded_global_alpha(self.amax_x, self.amax_w, TARGET, TARGET)
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
        if time_gemm:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        if self.path == "fp4":
            y = ops.gemm_fp4_operands(xq, wq, snap=True, alpha=alpha, out_dtype=torch.bfloat16)
        else:
            y = ops.gemm_issue_rz(xq, wq, snap=True, alpha=alpha, out_dtype=torch.bfloat16)
        if time_gemm:
            stop.record()
            self.gemm_events.append((start, stop))
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
    random codes: a measured library figure beside the roofline (this pool's peak file has no FP4
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


def _linear_step(torch, device, steps: int = 10) -> dict | None:
    """Forward + backward of one UE5M3Linear of the benchmark shape (X 8192x4096, W 21504x4096,
    bf16, default recipe: dY stochastic, W 2-D tiles): three GEMMs and six operand
    quantizations per step.  Reported beside the headline, not part of it."""

    from ue5m3_fp4.nn import UE5M3Linear

    try:
        layer = UE5M3Linear(K, N, bias=False, backend="probe_matched", module_name="layers.0.mixer.up_proj",
                            device=device, dtype=torch.bfloat16)
        g = torch.Generator().manual_seed(3)
        with torch.no_grad():
            layer.weight.copy_((0.02 * torch.randn(N, K, generator=g)).to(torch.bfloat16))
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(device).requires_grad_(True)
        dy = (1e-3 * torch.randn(M, N, generator=g)).to(torch.bfloat16).to(device)
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
        return {"what": "UE5M3Linear forward + backward, tokens 8192, in 4096, out 21504, bf16",
                "ms": ms, "tflops": 3 * 2.0 * M * N * K / (ms * 1e-3) / 1e12, "steps": steps}
    except Exception as error:  # noqa: BLE001 - informational leg
        return {"error": f"{type(error).__name__}: {error}"[:200]}


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

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # samples cover warm-up (same work) and the timed region
    for _ in range(max(args.warmup, 3)):
        hot.step()
    from ue5m3_fp4 import _native

    launches_before = _native.launch_count
    hot.step_index = 0
    sampler.mark()
    seconds = _timed(torch, dist, world, lambda: hot.step(time_gemm=True), args.steps)
    sampler.mark()
    clocks = sampler.stop() if rank == 0 else None
    launches = _native.launch_count - launches_before  # kernels of the library inside the timed region
    b200.check_gemm_status(device)
    gemm_s = sum(a.elapsed_time(b) for a, b in hot.gemm_events) / len(hot.gemm_events) / 1e3

    for _ in range(2):
        hot.step_e2e()
    e2e_seconds = _timed(torch, dist, world, hot.step_e2e, args.steps, finish=hot.finish_e2e)

    flops_per_rank = 2.0 * M * N * K
    value = flops_per_rank * world * args.steps / seconds / 1e12
    e2e_value = flops_per_rank * world * args.steps / e2e_seconds / 1e12
    if rank == 0:
        quant = _quantize_headline(torch, b200, device, max(args.steps, 40), peaks)
        cpu = cpu_baseline() if world == 1 else None
        bf16_peak = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
        fp4 = hot.path == "fp4"
        # The FP4 kernel issues kind::mxf4nvf4 MMAs, four times the BF16 MMA rate of the same
        # tensor core; its denominator is 4 x the measured cuBLAS BF16 figure (no FP4 peak is
        # measured on this pool; the nominal dense FP4 figure is 9000 TFLOP/s).
        peak_tf = 4.0 * bf16_peak if fp4 else bf16_peak
        achieved = flops_per_rank / gemm_s / 1e12
        gemm_kernel = ("gemm_fp4_pair_kernel" if os.environ.get("UE5M3_FP4_CTA_PAIR", "1") != "0" else "gemm_fp4_kernel") \
            if fp4 else "gemm_issue_rz_kernel"
        library_tf = _library_fp4_reference(torch, device) if fp4 else None
        linear = _linear_step(torch, device) if world == 1 else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": seconds / args.steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": ("fp4 (e2m1 x ue5m3->ue4m3 block scales) tensor-core MMA, fp32 accumulate" if fp4
                      else "fp4(e2m1)xue5m3 codes as encoded bf16 -> fp32 RZ accumulate"),
            "data": "synthetic", "config": {**_config(world), "gemm_kernel": gemm_kernel},
            "roofline": {
                "kernel": gemm_kernel, "bound": "tensor",
                "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                # DRAM bytes per launch: ncu capture of the M4096 N8192 case (reads 1.03 x the operand
                # bytes) scaled by the operand bytes of this shape, plus the bf16 output once
                "traffic": (1.03 * (M * K / 2 + N * K / 2 + (M + N) * K / 16) + M * N * 2) if fp4 else None,
                "peak_source": (f"4 x {peaks['source']} cuBLAS bf16 sustained ({bf16_peak}); nominal dense FP4 9000"
                                if fp4 else f"{peaks['source']} cuBLAS bf16 sustained (burst {peaks['bf16_tflops']})"),
                "frac_of_nominal_fp4_9000": achieved / 9000.0,
                "library_reference": (None if library_tf is None else {
                    "what": "cuBLASLt NVFP4 GEMM via torch._scaled_mm, same shape, random codes, 20 launches",
                    "tflops": library_tf, "frac": achieved / library_tf}),
                "algorithmic_flops_per_launch": flops_per_rank, "gemm_ms": gemm_s * 1e3,
            },
            "quantize": quant,
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_seconds / args.steps * 1e3,
                    "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2,
                    "note": "every step: X from pinned host memory in, bf16 Y to pinned host memory out (W resident); the two copy directions run on their own streams and overlap the neighbouring steps"},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if linear is not None:
            line["linear_step"] = linear
        if cpu is not None:
            line["cpu_baseline"] = cpu
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
    parser.add_argument("--case", default=None, choices=["gemm-small", "gemm-fp4-small", "quantize", "linear-step"],
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
