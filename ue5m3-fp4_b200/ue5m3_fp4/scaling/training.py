"""Periodic sample-and-hold tensor scaling for training (D-step delayed amax).

API and semantics of the reference's ``scaling/training.py``: ``sample_global_amax``
(training.py:18-79) and ``TrainingScaleState`` (training.py:90-216).  The sample itself
is the single-pass device reduction of the sm_100a library; the result stays on the
device and is MAX all-reduced across the data-parallel ranks of the default process
group (NCCL over NVLink when the group is NCCL).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist
from torch import Tensor

from ue5m3_fp4.recipe import OperandRole, UE5M3Recipe


def _local_amax(tensor: Tensor) -> Tensor:
    """fp32 0-dim amax of the local data on its device, by the native kernel."""

    from ue5m3_fp4.backends import b200

    to_local = getattr(tensor, "to_local", None)
    if callable(to_local):  # sharded DTensor: reduce the local shard, MAX across ranks below
        tensor = to_local()
    if not tensor.is_cuda:
        raise RuntimeError(
            "tensor amax sampling runs on the B200 kernels and requires a CUDA tensor; "
            "there is no CPU path"
        )
    if tensor.dtype not in (torch.bfloat16, torch.float32):
        tensor = tensor.to(torch.float32)
    return b200.tensor_amax(tensor)


def sample_global_amax(tensor: Tensor, *, label: str) -> Tensor:
    """Finite FP32 amax of ``tensor``, synchronised over the default process group."""

    if not isinstance(tensor, Tensor):
        raise TypeError("tensor must be a torch.Tensor")
    if not isinstance(label, str) or not label:
        raise ValueError("label must be a non-empty string")
    if not tensor.is_floating_point():
        raise TypeError("tensor must have a floating-point dtype")
    if tensor.numel() == 0:
        raise ValueError(f"cannot sample {label} from an empty tensor")
    if tensor.device.type == "meta":
        raise RuntimeError(f"cannot sample {label} from a meta tensor")

    value = _local_amax(tensor.detach()).to(dtype=torch.float32).reshape(())
    if not bool(torch.isfinite(value)):
        raise ValueError(f"cannot sample {label} from non-finite values")

    if not dist.is_available() or not dist.is_initialized():
        return value
    try:
        world_size = dist.get_world_size()
    except (RuntimeError, ValueError) as error:
        raise RuntimeError(f"cannot determine process-group size for {label}") from error
    if world_size < 1:
        raise RuntimeError(f"process-group size for {label} must be positive, got {world_size}")
    if world_size == 1:
        return value
    try:
        backend = str(dist.get_backend()).lower()
    except (RuntimeError, ValueError) as error:
        raise RuntimeError(f"cannot determine collective backend for {label}") from error
    if "nccl" in backend and value.device.type != "cuda":
        raise RuntimeError(
            f"global {label} synchronization uses NCCL but its scalar is on "
            f"{value.device.type!r}, not CUDA"
        )
    synchronized = value.clone()
    try:
        dist.all_reduce(synchronized, op=dist.ReduceOp.MAX)
    except (RuntimeError, ValueError) as error:
        raise RuntimeError(f"failed to synchronize global {label} with a MAX collective") from error
    if not bool(torch.isfinite(synchronized)):
        raise RuntimeError(f"global {label} MAX collective returned a non-finite value")
    return synchronized


@dataclass(slots=True)
class _ScaleEntry:
    reference: Tensor
    last_refresh_step: int
    refreshes: int = 1
    reuses: int = 0


class TrainingScaleState:
    """Process-local held tensor amaxes, keyed by (operand role, module name).

    ``begin_step`` is called once per optimizer step.  A key refreshes on first use
    and whenever ``step - last_refresh_step >= D``; in between the sampled value is
    held unchanged (no window, no rolling maximum).  Nothing is checkpointed.
    """

    def __init__(self, recipe: UE5M3Recipe) -> None:
        if not isinstance(recipe, UE5M3Recipe):
            raise TypeError("recipe must be a UE5M3Recipe")
        self.recipe = recipe
        self._step: int | None = None
        self._entries: dict[tuple[OperandRole, str], _ScaleEntry] = {}
        self._begin_step_calls = 0

    @property
    def step(self) -> int | None:
        return self._step

    def begin_step(self, step: int) -> None:
        if type(step) is not int or step < 1:
            raise ValueError("step must be a positive integer")
        if self._step is not None and step <= self._step:
            raise ValueError(f"training steps must increase strictly; current={self._step}, got={step}")
        self._step = step
        self._begin_step_calls += 1

    @staticmethod
    def _sample_amax(tensor: Tensor) -> Tensor:
        return sample_global_amax(tensor, label="training operand amax")

    def reference(self, role: str, module_name: str, tensor: Tensor) -> Tensor:
        """The held amax of (role, module) as a fresh 0-dim fp32 tensor."""

        if self._step is None:
            raise RuntimeError("begin_step(step) must be called before reference()")
        normalized = self.recipe.normalize_role(role)
        if not isinstance(module_name, str) or not module_name:
            raise ValueError("module_name must be a non-empty string")
        if not isinstance(tensor, Tensor):
            raise TypeError("tensor must be a torch.Tensor")
        key = (normalized, module_name)
        entry = self._entries.get(key)
        if entry is None:
            self._entries[key] = entry = _ScaleEntry(self._sample_amax(tensor), self._step)
        elif self._step - entry.last_refresh_step >= self.recipe.delayed_scale_interval:
            entry.reference = self._sample_amax(tensor)
            entry.last_refresh_step = self._step
            entry.refreshes += 1
        else:
            if entry.reference.device != tensor.device:
                raise RuntimeError(
                    "tensor device changed while a delayed reference was held; "
                    "create a new TrainingScaleState for the new runtime"
                )
            entry.reuses += 1
        # Callers get a copy, so in-place edits cannot corrupt the held value.
        return entry.reference.clone()

    def state_dict(self) -> dict[str, Any]:
        return {}

    def clear_runtime(self) -> int:
        cleared = len(self._entries)
        self._entries.clear()
        self._step = None
        self._begin_step_calls = 0
        return cleared

    def report(self) -> dict[str, Any]:
        ordered = sorted(self._entries.items(), key=lambda item: (item[0][0].value, item[0][1]))
        return {
            "schema": "ue5m3_fp4_training_scale_state_v1",
            "policy": "periodic_sample_and_hold",
            "rolling_or_window_maximum": False,
            "refresh_interval_steps": self.recipe.delayed_scale_interval,
            "current_step": self._step,
            "begin_step_calls": self._begin_step_calls,
            "checkpoint_cache_entries": 0,
            "entries": [
                {
                    "role": role.value,
                    "module_name": module_name,
                    "reference_amax": float(entry.reference.detach().cpu().item()),
                    "last_refresh_step": entry.last_refresh_step,
                    "refreshes": entry.refreshes,
                    "reuses": entry.reuses,
                }
                for (role, module_name), entry in ordered
            ],
        }


__all__ = ["TrainingScaleState", "sample_global_amax"]
