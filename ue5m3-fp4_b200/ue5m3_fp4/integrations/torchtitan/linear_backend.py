"""Backend seam of the TorchTitan adapter (reference integrations/torchtitan/linear_backend.py:17-62)."""

from __future__ import annotations

from collections.abc import Callable

from torch import nn

from ue5m3_fp4.nn.convert import ConversionRecord, convert_linear_modules
from ue5m3_fp4.nn.linear import LinearBackend, normalize_linear_backend
from ue5m3_fp4.recipe import UE5M3Recipe
from ue5m3_fp4.scaling.training import TrainingScaleState

LINEAR_BACKEND_NAME = LinearBackend.PROBE_MATCHED_TRITON.value
LINEAR_BACKEND_PROBE_MATCHED = True
_MARKER = "_ue5m3_reported_internal_linear"


def convert_reported_linears(
    model: nn.Module,
    *,
    recipe: UE5M3Recipe,
    scale_state: TrainingScaleState,
    selector: Callable[[str, nn.Linear], bool],
    backend: str | LinearBackend = LinearBackend.PROBE_MATCHED_TRITON,
) -> tuple[ConversionRecord, ...]:
    """Convert the selected linears and tag each replacement with the backend that owns it."""

    resolved = normalize_linear_backend(backend)
    records = convert_linear_modules(model, recipe=recipe, scale_state=scale_state, backend=resolved, selector=selector)
    for record in records:
        setattr(model.get_submodule(record.module_name), _MARKER, resolved.value)
    return records


def is_reported_quantized_linear(module: object) -> bool:
    return isinstance(module, nn.Module) and isinstance(getattr(module, _MARKER, None), str)


__all__ = ["LINEAR_BACKEND_NAME", "LINEAR_BACKEND_PROBE_MATCHED", "convert_reported_linears", "is_reported_quantized_linear"]
