from ue5m3_fp4.scaling.inference import FP4InferenceScalingController
from ue5m3_fp4.scaling.training import TrainingScaleState

__all__ = ["FP4InferenceScalingController", "TrainingScaleState"]
