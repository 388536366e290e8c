"""Periodic sample-and-hold tensor scaling for training (D-step delayed amax).

API and semantics of the reference's ``scaling/training.py``: ``sample_global_amax``
(training.py:18-79) and ``TrainingScaleState`` (training.py:90-216).

What differs is where the work happens.  A sample is ONE pass of the sm_100a reduction
kernel, its result stays on the device, and the MAX all-reduce over the data-parallel
ranks (NCCL over NVLink) runs on that device scalar in stream order.  The reference looks
at every sample on the host twice (``bool(torch.isfinite(...))`` before and after the
collective, training.py:47,77), i.e. 672 pipeline drains on a refresh step of the
112-linear model.  ``TrainingScaleState`` instead keeps the sampled scalars of a step in a
list and tests them all with one device reduction and one host read when the NEXT step
begins (or when ``verify_samples`` / ``report`` is called): a non-finite sample still stops
the run with the reference's error, one step later, and the steps in between cost no
synchronisation.  ``sample_weights`` takes the amaxes of many weights (they do not depend on
the activations) before the forward pass and reduces them across ranks with a single
collective.  The public ``sample_global_amax`` keeps the reference's immediate check.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Iterable

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


def _check_sample_source(tensor: Tensor, label: str) -> None:
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


def _group_size(label: str) -> int:
    """Ranks of the default process group (1 without one), with the reference's errors."""

    if not dist.is_available() or not dist.is_initialized():
        return 1
    try:
        world_size = dist.get_world_size()
    except (RuntimeError, ValueError) as error:
        raise RuntimeError(f"cannot determine process-group size for {label}") from error
    if world_size < 1:
        raise RuntimeError(f"process-group size for {label} must be positive, got {world_size}")
    return world_size


def _max_over_ranks(value: Tensor, label: str) -> Tensor:
    """In-place MAX all-reduce of a device tensor over the default group."""

    try:
        backend = str(dist.get_backend()).lower()
    except (RuntimeError, ValueError) as error:
        raise RuntimeError(f"cannot determine collective backend for {label}") from error
    if "nccl" in backend and value.device.type != "cuda":
        raise RuntimeError(
            f"global {label} synchronization uses NCCL but its scalar is on "
            f"{value.device.type!r}, not CUDA"
        )
    try:
        dist.all_reduce(value, op=dist.ReduceOp.MAX)
    except (RuntimeError, ValueError) as error:
        raise RuntimeError(f"failed to synchronize global {label} with a MAX collective") from error
    return value


def _sample_on_device(tensor: Tensor, label: str) -> Tensor:
    """Local kernel reduction + MAX over the ranks; the result is never looked at on the host."""

    _check_sample_source(tensor, label)
    value = _local_amax(tensor.detach()).to(dtype=torch.float32).reshape(())
    if _group_size(label) > 1:
        value = _max_over_ranks(value.clone(), label)
    return value


def sample_global_amax(tensor: Tensor, *, label: str) -> Tensor:
    """Finite FP32 amax of ``tensor``, synchronised over the default process group; raises at
    once on a non-finite value, as the reference does (one host read for that)."""

    _check_sample_source(tensor, label)
    local = _local_amax(tensor.detach()).to(dtype=torch.float32).reshape(())
    if _group_size(label) == 1:
        if not bool(torch.isfinite(local)):
            raise ValueError(f"cannot sample {label} from non-finite values")
        return local
    # Every rank joins the collective, also one whose own sample is not finite (it sends +inf),
    # so that no rank is left waiting; one host read afterwards tells the two errors apart.
    synchronized = _max_over_ranks(torch.nan_to_num(local, nan=float("inf")).clone(), label)
    local_ok, global_ok = torch.stack((torch.isfinite(local), torch.isfinite(synchronized))).tolist()
    if not local_ok:
        raise ValueError(f"cannot sample {label} from non-finite values")
    if not global_ok:
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
        self._unverified: list[tuple[str, Tensor]] = []

    @property
    def step(self) -> int | None:
        return self._step

    def begin_step(self, step: int) -> None:
        if type(step) is not int or step < 1:
            raise ValueError("step must be a positive integer")
        if self._step is not None and step <= self._step:
            raise ValueError(f"training steps must increase strictly; current={self._step}, got={step}")
        self.verify_samples()
        self._poll_kernels()
        self._step = step
        self._begin_step_calls += 1

    def verify_samples(self) -> None:
        """Host check of every amax sampled since the last check: one device reduction, one
        read.  Raises the reference's error for the first non-finite sample."""

        pending, self._unverified = self._unverified, []
        if not pending:
            return
        by_device: dict[torch.device, list[tuple[str, Tensor]]] = {}
        for name, value in pending:
            by_device.setdefault(value.device, []).append((name, value))
        for group in by_device.values():
            finite = torch.isfinite(torch.stack([value.reshape(()) for _, value in group]))
            if bool(finite.all()):
                continue
            bad = [name for (name, _), ok in zip(group, finite.tolist()) if not ok]
            raise ValueError(f"cannot sample training operand amax from non-finite values ({', '.join(bad)})")

    def _poll_kernels(self) -> None:
        devices = {entry.reference.device for entry in self._entries.values() if entry.reference.is_cuda}
        if devices:
            from ue5m3_fp4.backends import b200

            for device in devices:
                b200.poll_gemm_status(device)

    def _sample_amax(self, tensor: Tensor, name: str = "training operand amax") -> Tensor:
        value = _sample_on_device(tensor, "training operand amax")
        self._unverified.append((name, value))
        return value

    def _due(self, key: tuple[OperandRole, str]) -> bool:
        entry = self._entries.get(key)
        return entry is None or self._step - entry.last_refresh_step >= self.recipe.delayed_scale_interval

    def _store(self, key: tuple[OperandRole, str], value: Tensor) -> None:
        entry = self._entries.get(key)
        if entry is None:
            self._entries[key] = _ScaleEntry(value, self._step)
        else:
            entry.reference = value
            entry.last_refresh_step = self._step
            entry.refreshes += 1

    def sample_weights(self, weights: Iterable[tuple[str, Tensor]]) -> int:
        """Refreshes every WEIGHT reference that is due at the current step, all at once: one
        reduction kernel per weight into one vector, ONE MAX all-reduce for the vector.  Weights
        do not depend on the step's activations, so this can run before the forward pass; the
        ``reference("weight", ...)`` calls of the linears then find their values held.  Returns
        the number of weights sampled."""

        if self._step is None:
            raise RuntimeError("begin_step(step) must be called before sample_weights()")
        role = self.recipe.normalize_role("weight")
        due = [(name, tensor) for name, tensor in weights if self._due((role, name))]
        if not due:
            return 0
        for name, tensor in due:
            _check_sample_source(tensor, "training operand amax")
        values = torch.stack([_local_amax(tensor.detach()).to(torch.float32).reshape(()) for _, tensor in due])
        if _group_size("training operand amax") > 1:
            values = _max_over_ranks(values, "training operand amax")
        for index, (name, _) in enumerate(due):
            value = values[index].clone()
            self._unverified.append((f"weight:{name}", value))
            self._store((role, name), value)
        return len(due)

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
        if self._due(key):
            self._store(key, self._sample_amax(tensor, f"{normalized.value}:{module_name}"))
        else:
            entry = self._entries[key]
            if entry.reference.device != tensor.device:
                raise RuntimeError(
                    "tensor device changed while a delayed reference was held; "
                    "create a new TrainingScaleState for the new runtime"
                )
            entry.reuses += 1
        # Callers get a copy, so in-place edits cannot corrupt the held value.
        return self._entries[key].reference.clone()

    def state_dict(self) -> dict[str, Any]:
        return {}

    def clear_runtime(self) -> int:
        cleared = len(self._entries)
        self._entries.clear()
        self._unverified.clear()
        self._step = None
        self._begin_step_calls = 0
        return cleared

    def report(self) -> dict[str, Any]:
        self.verify_samples()
        ordered = sorted(self._entries.items(), key=lambda item: (item[0][0].value, item[0][1]))
        values = [entry.reference.detach().reshape(()).to(torch.float32) for _, entry in ordered]
        # one read for the whole table
        host = torch.stack([value.to(values[0].device) for value in values]).tolist() if values else []
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
                    "reference_amax": float(value),
                    "last_refresh_step": entry.last_refresh_step,
                    "refreshes": entry.refreshes,
                    "reuses": entry.reuses,
                }
                for ((role, module_name), entry), value in zip(ordered, host)
            ],
        }


__all__ = ["TrainingScaleState", "sample_global_amax"]
