"""UE5M3/E2M1 block-scaled FP4 quantization and the probe-matched GEMM on B200 (sm_100a).

Public names follow the reference package ``ue5m3_fp4`` so that its callers
(the TorchTitan Nemotron-H converter among them) import this package unchanged.
"""

from ue5m3_fp4.formats import E2M1, UE5M3, quantize_dequantize_blocks
from ue5m3_fp4.recipe import UE5M3Recipe
from ue5m3_fp4.scaling.inference import FP4InferenceScalingController
from ue5m3_fp4.scaling.training import TrainingScaleState

__all__ = [
    "E2M1",
    "UE5M3",
    "FP4InferenceScalingController",
    "TrainingScaleState",
    "UE5M3Recipe",
    "quantize_dequantize_blocks",
]
