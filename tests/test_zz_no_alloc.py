"""The allocation-free amax entry point (ue5m3_amax_static) against ue5m3_amax.

For hosts that cannot allocate device memory themselves - a C/C++ plugin whose device
memory all belongs to another runtime's pool, or a thread that must not pay for
cudaMalloc's device-wide synchronisation - the library keeps the reduction scratch in a
fixed array of its own.  This test calls that entry point through the C ABI twice in a row
(the array is shared and keeps the previous call's contents) and requires the very same
fp32 result as the entry point that takes caller-provided scratch.  Collected last on
purpose, so a failure here cannot hide another test's result in a run that stops at the
first failure.
"""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, native, x: torch.Tensor) -> tuple[float, float]:
    device = x.device
    with_scratch = torch.empty((), dtype=torch.float32, device=device)
    scratch = torch.zeros(lib.ue5m3_amax_scratch_bytes(), dtype=torch.uint8, device=device)
    static = torch.full((), -1.0, dtype=torch.float32, device=device)
    stream = native.stream_ptr(device)
    code = native.dtype_code(x.dtype)
    native.check(lib.ue5m3_amax(x.data_ptr(), code, x.numel(), with_scratch.data_ptr(), scratch.data_ptr(),
                                scratch.numel(), stream), "ue5m3_amax")
    native.check(lib.ue5m3_amax_static(x.data_ptr(), code, x.numel(), static.data_ptr(), stream),
                 "ue5m3_amax_static")
    torch.cuda.synchronize()
    return with_scratch.item(), static.item()


def test_static_scratch_amax_equals_caller_scratch_amax_twice_in_a_row():
    from ue5m3_fp4 import _native as native

    lib = native.load()
    g = torch.Generator().manual_seed(17)
    first = (torch.randn(8192 * 1024 + 13, generator=g) * 3.0).to(torch.bfloat16).cuda()
    second = torch.randn(300_001, generator=g).cuda()  # fp32, smaller grid than the first call
    for tensor in (first, second, first[5:]):
        expected, got = _both(lib, native, tensor)
        assert got == expected == tensor.float().abs().max().item()


def test_static_scratch_amax_allocates_no_device_memory():
    """What the entry point is for: neither the driver's free-memory figure nor torch's
    allocator moves across calls (after the first call on the device, which only looks up the
    address of the library's own array)."""

    from ue5m3_fp4 import _native as native

    lib = native.load()
    x = torch.randn(1 << 22, device="cuda")
    out = torch.zeros((), dtype=torch.float32, device="cuda")
    stream = native.stream_ptr(x.device)
    native.check(lib.ue5m3_amax_static(x.data_ptr(), 1, x.numel(), out.data_ptr(), stream), "ue5m3_amax_static")
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    allocated_before, reserved_before = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for _ in range(3):
        native.check(lib.ue5m3_amax_static(x.data_ptr(), 1, x.numel(), out.data_ptr(), stream), "ue5m3_amax_static")
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free_before   # nothing was taken from the device
    assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == (allocated_before, reserved_before)
    assert out.item() == x.abs().max().item()


def test_static_scratch_amax_rejects_oversized_and_bad_arguments():
    from ue5m3_fp4 import _native as native

    lib = native.load()
    x = torch.ones(16, device="cuda")
    out = torch.zeros((), device="cuda")
    assert lib.ue5m3_amax_static(x.data_ptr(), 1, (1 << 32) + 1, out.data_ptr(), None) == 8
    assert b"2^32" in lib.ue5m3_last_cuda_error()
    assert lib.ue5m3_amax_static(None, 1, 16, out.data_ptr(), None) == 1
    assert lib.ue5m3_amax_static(x.data_ptr(), 5, 16, out.data_ptr(), None) == 1
