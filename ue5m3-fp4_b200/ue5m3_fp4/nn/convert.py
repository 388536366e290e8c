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


@dataclass(frozen=True)
class ProductPlan:
    """One of the three GEMMs of a converted linear on the FP4 tensor-core path."""

    module_name: str
    product: str                 # "forward", "data_gradient" or "weight_gradient"
    m: int
    n: int
    k: int
    packed_operands: bool        # K % 64 == 0: both operands leave the one-launch operand quantizers
    weight_in_one_launch: bool   # forward / data gradient: W and W^T come from one read of the weight
    workspace_bytes: int         # what the recomputation pass wants for this product


def plan_fp4_products(records, tokens: int) -> tuple[ProductPlan, ...]:
    """What a step of ``tokens`` tokens asks of the device for every converted linear: the three
    products Y = X W^T [tokens, out, in], dX = dY W [tokens, in, out] and dW = dY^T X
    [out, in, tokens] with the operand constraints of the packed path (reduction axis a
    multiple of 64) and the recomputation pass's workspace.  Has no counterpart in the
    reference, whose Triton path has neither packed operands nor a workspace."""

    from ue5m3_fp4.backends import b200

    if tokens <= 0:
        raise ValueError("tokens must be positive")
    plans = []
    for record in records:
        both = record.in_features % 64 == 0 and record.out_features % 64 == 0
        for product, (m, n, k) in (
            ("forward", (tokens, record.out_features, record.in_features)),
            ("data_gradient", (tokens, record.in_features, record.out_features)),
            ("weight_gradient", (record.out_features, record.in_features, tokens)),
        ):
            plans.append(ProductPlan(record.module_name, product, m, n, k, k % 64 == 0,
                                     both and product != "weight_gradient", b200.fallback_workspace_bytes(m, n, k)))
    return tuple(plans)


def reserve_device_workspace(records, tokens: int, device: torch.device) -> int:
    """Size the recomputation pass's per-stream workspace for the largest product of the
    converted linears now, on ``device``'s current stream, so that no training step grows it.
    Returns the number of bytes held."""

    from ue5m3_fp4.backends import b200

    need = max((plan.workspace_bytes for plan in plan_fp4_products(records, tokens)), default=0)
    return b200.reserve_fallback_workspace(device, need)


__all__ = [
    "ConversionRecord",
    "LinearSelector",
    "ProductPlan",
    "convert_linear_modules",
    "exclude_lm_head",
    "plan_fp4_products",
    "reserve_device_workspace",
    "select_all_linears",
]
