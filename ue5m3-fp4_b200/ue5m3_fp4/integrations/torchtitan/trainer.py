"""Once-per-optimizer-step bridge between a trainer and the D=50 scale states
(reference integrations/torchtitan/trainer.py:19-88)."""

from __future__ import annotations

from collections.abc import Iterable
from functools import wraps
from typing import Any

from torch import nn

from ue5m3_fp4.scaling.training import TrainingScaleState

_HOOK_MARKER = "_ue5m3_fp4_logical_step_hook_v1"


def training_scale_states(model_parts: Iterable[nn.Module]) -> tuple[TrainingScaleState, ...]:
    found: dict[int, TrainingScaleState] = {}
    for part in model_parts:
        if not isinstance(part, nn.Module):
            raise TypeError("every model part must be a torch.nn.Module")
        for module in part.modules():
            state = getattr(module, "scale_state", None)
            if isinstance(state, TrainingScaleState):
                found.setdefault(id(state), state)
    return tuple(found.values())


def begin_training_step(model_parts: Iterable[nn.Module], step: int) -> int:
    """Advance every distinct scale state to `step`; models without FP4 linears are a no-op.

    On a step at which weight references are due (1, 51, 101, ... with D = 50) the amaxes of
    all FP4 linears' weights that share a state are then sampled together - they do not depend
    on the step's activations - and reduced across the data-parallel ranks with ONE collective
    (``TrainingScaleState.sample_weights``) instead of one per linear inside the forward pass."""

    if type(step) is not int or step < 1:
        raise ValueError("step must be a positive integer")
    parts = list(model_parts)
    states = training_scale_states(parts)
    for state in states:
        if state.step is not None and state.step >= step:
            raise RuntimeError(
                f"TorchTitan UE5M3 step hook was called out of order: state={state.step}, trainer={step}"
            )
        state.begin_step(step)
    weights: dict[int, list] = {}
    for part in parts:
        for module in part.modules():
            state = getattr(module, "scale_state", None)
            name, weight = getattr(module, "module_name", None), getattr(module, "weight", None)
            if isinstance(state, TrainingScaleState) and isinstance(name, str) and weight is not None and weight.is_cuda:
                weights.setdefault(id(state), []).append((name, weight.detach()))
    for state in states:
        state.sample_weights(weights.get(id(state), ()))
    return len(states)


def install_trainer_step_hook(trainer_cls: type[Any] | None = None) -> type[Any]:
    """Wrap ``Trainer.train_step`` so the sample-and-hold lifecycle advances once per optimizer
    step (not per gradient-accumulation micro-batch).  Idempotent."""

    if trainer_cls is None:
        try:
            from torchtitan.train import Trainer
        except ImportError as error:
            raise ImportError("TorchTitan is required; install the pinned upstream revision") from error
        trainer_cls = Trainer
    original = getattr(trainer_cls, "train_step", None)
    if not callable(original):
        raise TypeError("trainer class must expose a callable train_step")
    if getattr(original, _HOOK_MARKER, False):
        return trainer_cls

    @wraps(original)
    def train_step(self: Any, *args: Any, **kwargs: Any) -> Any:
        parts = getattr(self, "model_parts", None)
        if parts is None:
            raise RuntimeError("TorchTitan Trainer has no model_parts at train_step")
        begin_training_step(parts, getattr(self, "step", None))
        return original(self, *args, **kwargs)

    setattr(train_step, _HOOK_MARKER, True)
    trainer_cls.train_step = train_step
    return trainer_cls


__all__ = ["begin_training_step", "install_trainer_step_hook", "training_scale_states"]
