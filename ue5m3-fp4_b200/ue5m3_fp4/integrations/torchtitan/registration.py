"""Registration of the UE5M3 model converters and the logical-step hook with TorchTitan's
public extension points (reference integrations/torchtitan/registration.py:31-155).

The converter names are the reference's, so ``model.converters=["ue5m3_fp4.reported_b16_d50"]``
and ``experimental.custom_import="ue5m3_fp4.integrations.torchtitan.plugin"`` keep working.
The Nemotron-H TrainSpec, data loader and Transformer-Engine comparators of the reference are
not registered here; they are outside this package.
"""

from __future__ import annotations

from dataclasses import replace
from typing import Any

from torch import nn

from ue5m3_fp4.integrations.torchtitan.selection import convert_reported_nemotron_h
from ue5m3_fp4.integrations.torchtitan.trainer import install_trainer_step_hook
from ue5m3_fp4.nn.linear import LinearBackend
from ue5m3_fp4.recipe import UE5M3Recipe

CONVERTER_B16_NAME = "ue5m3_fp4.reported_b16_d50"
CONVERTER_B32_NAME = "ue5m3_fp4.reported_b32_d50"
CONVERTER_TORCH_CONTROL_NAME = "ue5m3_fp4.torch_control_b16_d50"
CONVERTER_NAME = CONVERTER_B16_NAME

_registered = False


class ReportedUE5M3Converter:
    """TorchTitan ``ModelConverter`` for the reported B=16, D=50 placement."""

    def __init__(self, _job_config: Any, _parallel_dims: Any) -> None:
        self.conversion = None

    def convert(self, model: nn.Module) -> None:
        self.conversion = convert_reported_nemotron_h(model)

    def post_optimizer_hook(self, _model: nn.Module | list[nn.Module]) -> None:
        return None


class ReportedUE5M3B32Converter(ReportedUE5M3Converter):
    def convert(self, model: nn.Module) -> None:
        recipe = replace(UE5M3Recipe.proposed(), name="proposed_ue5m3_b32_d50", block_size=32)
        self.conversion = convert_reported_nemotron_h(model, recipe=recipe)


class UE5M3TorchControlConverter(ReportedUE5M3Converter):
    def convert(self, model: nn.Module) -> None:
        self.conversion = convert_reported_nemotron_h(model, backend=LinearBackend.TRITON_QUANT_TORCH)


def register_torchtitan() -> None:
    """Register converters and install the step hook exactly once."""

    global _registered
    if _registered:
        return
    try:
        from torchtitan.protocols.model_converter import register_model_converter
    except ImportError as error:
        raise ImportError("TorchTitan is required to register the UE5M3 converters") from error
    register_model_converter(ReportedUE5M3Converter, CONVERTER_B16_NAME)
    register_model_converter(ReportedUE5M3B32Converter, CONVERTER_B32_NAME)
    register_model_converter(UE5M3TorchControlConverter, CONVERTER_TORCH_CONTROL_NAME)
    install_trainer_step_hook()
    _registered = True


__all__ = [
    "CONVERTER_B16_NAME",
    "CONVERTER_B32_NAME",
    "CONVERTER_NAME",
    "CONVERTER_TORCH_CONTROL_NAME",
    "ReportedUE5M3B32Converter",
    "ReportedUE5M3Converter",
    "UE5M3TorchControlConverter",
    "register_torchtitan",
]
