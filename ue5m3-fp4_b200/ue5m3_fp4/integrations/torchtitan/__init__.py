"""TorchTitan boundary: converter registration, reported Nemotron-H selection of the 112
internal linears, FP32 output head, and the once-per-optimizer-step hook.

Only the boundary of the reference's ``integrations/torchtitan`` package is provided
(registration.py, linear_backend.py, selection.py, trainer.py, plugin.py); the Nemotron-H
model adapter, data loader, state-dict adapter and Transformer-Engine comparators are not
part of this package.
"""

from ue5m3_fp4.integrations.torchtitan.linear_backend import convert_reported_linears, is_reported_quantized_linear
from ue5m3_fp4.integrations.torchtitan.selection import (
    FP32OutputLinear,
    NemotronHSelectionError,
    ReportedConversion,
    convert_reported_nemotron_h,
    reported_projection,
    select_reported_nemotron_h_linear,
)
from ue5m3_fp4.integrations.torchtitan.trainer import begin_training_step, install_trainer_step_hook

__all__ = [
    "FP32OutputLinear",
    "NemotronHSelectionError",
    "ReportedConversion",
    "begin_training_step",
    "convert_reported_linears",
    "convert_reported_nemotron_h",
    "install_trainer_step_hook",
    "is_reported_quantized_linear",
    "reported_projection",
    "select_reported_nemotron_h_linear",
]
