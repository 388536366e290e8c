"""In-place replacement of selected ``torch.nn.Linear`` children by ``UE5M3Linear``.

Same contract as the reference's ``nn/convert.py:42-145``: an explicit selector is
required, only exact ``nn.Linear`` objects are converted (selected subclasses and
aliased module objects are rejected), every selector decision is taken before the
first mutation, the root is never replaced, and converted modules keep the original
``Parameter`` objects.
"""

from __future__ import annotations

from collections import defaultdict
from collections.abc import Callable
from dataclasses import dataclass

import torch

from ue5m3_fp4.nn.linear import LinearBackend, UE5M3Linear, normalize_linear_backend
from ue5m3_fp4.recipe import UE5M3Recipe
from ue5m3_fp4.scaling.training import TrainingScaleState

LinearSelector = Callable[[str, torch.nn.Linear], bool]


def select_all_linears(_module_name: str, _module: torch.nn.Linear) -> bool:
    return True


def exclude_lm_head(module_name: str, _module: torch.nn.Linear) -> bool:
    return module_name.rsplit(".", 1)[-1] != "lm_head"


@dataclass(frozen=True)
class ConversionRecord:
    module_name: str
    in_features: int
    out_features: int
    bias: bool


def convert_linear_modules(
    model: torch.nn.Module,
    *,
    recipe: UE5M3Recipe | None = None,
    scale_state: TrainingScaleState | None = None,
    backend: str | LinearBackend = LinearBackend.PROBE_MATCHED_TRITON,
    selector: LinearSelector | None = None,
) -> tuple[ConversionRecord, ...]:
    if not isinstance(model, torch.nn.Module):
        raise TypeError("model must be a torch.nn.Module")
    if isinstance(model, torch.nn.Linear):
        raise ValueError("convert_linear_modules cannot replace the model root")
    recipe = recipe or UE5M3Recipe.proposed()
    if not isinstance(recipe, UE5M3Recipe):
        raise TypeError("recipe must be a UE5M3Recipe")
    if scale_state is not None:
        if not isinstance(scale_state, TrainingScaleState):
            raise TypeError("scale_state must be a TrainingScaleState")
        if scale_state.recipe != recipe:
            raise ValueError("scale_state.recipe must match recipe")
    scale_state = scale_state or TrainingScaleState(recipe)
    resolved_backend = normalize_linear_backend(backend)
    if selector is None:
        raise ValueError(
            "selector is required; pass select_all_linears explicitly to convert every child linear"
        )
    if not callable(selector):
        raise TypeError("selector must be callable")

    linears = [
        (name, module)
        for name, module in model.named_modules(remove_duplicate=False)
        if name and isinstance(module, torch.nn.Linear)
    ]
    subclassed = [
        f"{name} ({type(module).__qualname__})"
        for name, module in linears
        if type(module) is not torch.nn.Linear and selector(name, module)
    ]
    if subclassed:
        raise TypeError(
            "Generic conversion supports exact nn.Linear modules only; "
            f"architecture-specific subclasses require an adapter: {', '.join(subclassed)}"
        )
    exact = [(name, module) for name, module in linears if type(module) is torch.nn.Linear]
    names_by_object: dict[int, list[str]] = defaultdict(list)
    for name, module in exact:
        names_by_object[id(module)].append(name)
    shared = [names for names in names_by_object.values() if len(names) > 1]
    if shared:
        rendered = "; ".join(", ".join(names) for names in shared)
        raise ValueError(
            f"Aliased nn.Linear module objects require architecture-specific conversion: {rendered}"
        )

    chosen = [(name, module) for name, module in exact if selector(name, module)]
    records = []
    for name, module in chosen:
        parent_name, _, child = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        replacement = UE5M3Linear.from_float(
            module, recipe=recipe, scale_state=scale_state, backend=resolved_backend, module_name=name
        )
        replacement.train(module.training)
        setattr(parent, child, replacement)
        records.append(ConversionRecord(name, module.in_features, module.out_features, module.bias is not None))
    return tuple(records)


__all__ = [
    "ConversionRecord",
    "LinearSelector",
    "convert_linear_modules",
    "exclude_lm_head",
    "select_all_linears",
]
