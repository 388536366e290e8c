"""Reported Nemotron-H 8B precision placement: exactly 112 internal FP4 linears and an
FP32 vocabulary head (reference integrations/torchtitan/selection.py:28-283).

The selector is architecture-specific on purpose: an unknown ``Linear`` is never silently
treated as part of the published experiment.
"""

from __future__ import annotations

import re
from dataclasses import dataclass, replace

import torch
from torch import nn
from torch.nn import functional as F

from ue5m3_fp4.integrations.torchtitan.linear_backend import convert_reported_linears
from ue5m3_fp4.nn.convert import ConversionRecord
from ue5m3_fp4.nn.linear import LinearBackend, normalize_linear_backend
from ue5m3_fp4.recipe import UE5M3Recipe
from ue5m3_fp4.scaling.training import TrainingScaleState

# M = Mamba2 mixer, * = self-attention, - = MLP
REPORTED_NEMOTRON_H_8B_PATTERN = "M-M-M-M*-M-M-M-M-M*-M-M-M-M-M*-M-M-M-M-M*-M-M-M-M-M-"
REPORTED_NEMOTRON_H_LAYER_COUNT = 52
REPORTED_ELIGIBLE_LINEAR_COUNT = 112
REPORTED_OUTPUT_HEAD_COUNT = 1

_PROJECTION = re.compile(
    r"(?:^|\.)layers\.(?P<layer>\d+)\.mixer\."
    r"(?P<projection>in_proj|out_proj|q_proj|k_proj|v_proj|o_proj|up_proj|down_proj)$"
)
_ALLOWED = {
    "M": frozenset({"in_proj", "out_proj"}),
    "*": frozenset({"q_proj", "k_proj", "v_proj", "o_proj"}),
    "-": frozenset({"up_proj", "down_proj"}),
}


class NemotronHSelectionError(RuntimeError):
    """The model does not match the reported 8B module layout."""


class FP32OutputLinear(nn.Linear):
    """Vocabulary head computed in FP32 on the original (shared) parameters."""

    @classmethod
    def from_float(cls, module: nn.Linear) -> FP32OutputLinear:
        if type(module) is not nn.Linear:
            raise TypeError("the FP32 output-head adapter expects an exact nn.Linear")
        head = cls(module.in_features, module.out_features, bias=module.bias is not None, device="meta",
                   dtype=module.weight.dtype)
        head.weight = module.weight
        if module.bias is not None:
            head.bias = module.bias
        head.train(module.training)
        return head

    def forward(self, inputs: torch.Tensor) -> torch.Tensor:
        with torch.autocast(device_type=inputs.device.type, enabled=False):
            bias = None if self.bias is None else self.bias.to(torch.float32)
            return F.linear(inputs.to(torch.float32), self.weight.to(torch.float32), bias)


def reported_projection(module_name: str) -> tuple[int, str] | None:
    """``(layer, projection)`` when the name is one of the 112 reported linears, else None."""

    if not isinstance(module_name, str):
        raise TypeError("module_name must be a string")
    found = _PROJECTION.search(module_name)
    if found is None:
        return None
    layer = int(found.group("layer"))
    if layer >= len(REPORTED_NEMOTRON_H_8B_PATTERN):
        return None
    projection = found.group("projection")
    return (layer, projection) if projection in _ALLOWED[REPORTED_NEMOTRON_H_8B_PATTERN[layer]] else None


def select_reported_nemotron_h_linear(module_name: str, _module: nn.Linear) -> bool:
    return reported_projection(module_name) is not None


def _output_head(model: nn.Module) -> tuple[str, nn.Linear]:
    heads = [
        (name, module)
        for name, module in model.named_modules(remove_duplicate=False)
        if name and name.rsplit(".", 1)[-1] in {"lm_head", "output"} and isinstance(module, nn.Linear)
        and ".mixer." not in name
    ]
    if len(heads) != REPORTED_OUTPUT_HEAD_COUNT:
        raise NemotronHSelectionError(
            "expected exactly one Nemotron-H vocabulary output head named "
            f"'lm_head' or 'output', found {[name for name, _ in heads]}"
        )
    name, module = heads[0]
    if type(module) is not nn.Linear:
        raise NemotronHSelectionError(f"output head {name!r} is {type(module).__qualname__}, expected nn.Linear")
    return name, module


def _check_architecture(model: nn.Module) -> None:
    config = getattr(model, "config", None) or getattr(getattr(model, "model", None), "config", None)
    if config is None:
        raise NemotronHSelectionError("Nemotron-H model does not expose a config")
    layers = getattr(config, "num_hidden_layers", None)
    if layers != REPORTED_NEMOTRON_H_LAYER_COUNT:
        raise NemotronHSelectionError(f"reported recipe requires 52 layers, model reports {layers!r}")
    if getattr(config, "hybrid_override_pattern", None) != REPORTED_NEMOTRON_H_8B_PATTERN:
        raise NemotronHSelectionError("model hybrid_override_pattern does not match the reported 8B architecture")


@dataclass(frozen=True, slots=True)
class ReportedConversion:
    fp4_linears: tuple[ConversionRecord, ...]
    fp32_output_head: str
    scale_state: TrainingScaleState
    linear_backend: str
    probe_matched_backend: bool


def convert_reported_nemotron_h(
    model: nn.Module,
    *,
    recipe: UE5M3Recipe | None = None,
    backend: str | LinearBackend = LinearBackend.PROBE_MATCHED_TRITON,
) -> ReportedConversion:
    """Apply the reported B=16 / B=32 precision placement in place."""

    if not isinstance(model, nn.Module):
        raise TypeError("model must be a torch.nn.Module")
    chosen = recipe or UE5M3Recipe.proposed()
    if chosen.block_size not in {16, 32}:
        raise ValueError("the reported TorchTitan converter requires block size 16 or 32")
    if chosen != replace(UE5M3Recipe.proposed(), name=chosen.name, block_size=chosen.block_size):
        raise ValueError(
            "the reported TorchTitan converter permits only the proposed recipe's block-16/block-32 variants"
        )
    resolved = normalize_linear_backend(backend)
    _check_architecture(model)
    head_name, head = _output_head(model)
    state = TrainingScaleState(chosen)
    records = convert_reported_linears(model, recipe=chosen, scale_state=state,
                                       selector=select_reported_nemotron_h_linear, backend=resolved)
    if len(records) != REPORTED_ELIGIBLE_LINEAR_COUNT:
        raise NemotronHSelectionError(
            "reported 8B conversion requires exactly 112 eligible internal linears; "
            f"converted {len(records)}: {[record.module_name for record in records]}"
        )
    parent_name, _, child = head_name.rpartition(".")
    setattr(model.get_submodule(parent_name) if parent_name else model, child, FP32OutputLinear.from_float(head))
    probe_matched = resolved is LinearBackend.PROBE_MATCHED_TRITON
    # plain attribute: nothing is added to the state dict
    model._ue5m3_reported_conversion = {
        "schema": "ue5m3_fp4_reported_nemotron_h_conversion_v1",
        "fp4_linear_count": len(records),
        "fp32_output_head": head_name,
        "linear_backend": resolved.value,
        "probe_matched_backend": probe_matched,
        "recipe": chosen.to_dict(),
    }
    return ReportedConversion(records, head_name, state, resolved.value, probe_matched)


__all__ = [
    "REPORTED_ELIGIBLE_LINEAR_COUNT",
    "REPORTED_NEMOTRON_H_8B_PATTERN",
    "REPORTED_NEMOTRON_H_LAYER_COUNT",
    "FP32OutputLinear",
    "NemotronHSelectionError",
    "ReportedConversion",
    "convert_reported_nemotron_h",
    "reported_projection",
    "select_reported_nemotron_h_linear",
]
