"""The TorchTitan boundary on CPU with synthetic fixtures (no real model), after the
reference's tests/test_exact_linear.py:142-250 and tests/test_torchtitan_trainer.py:21-97:
a 52-layer stand-in with 1x1 linears in the reported hybrid pattern converts to exactly 112
FP4 linears plus an FP32 head; the step hook advances the scale state once per optimizer step."""

from __future__ import annotations

import types

import pytest
import torch
from torch import nn

from ue5m3_fp4.integrations.torchtitan import (FP32OutputLinear, NemotronHSelectionError, begin_training_step,
                                               convert_reported_nemotron_h, install_trainer_step_hook,
                                               is_reported_quantized_linear, reported_projection)
from ue5m3_fp4.integrations.torchtitan.selection import REPORTED_NEMOTRON_H_8B_PATTERN
from ue5m3_fp4.nn import UE5M3Linear

_KINDS = {"M": ("in_proj", "out_proj"), "*": ("q_proj", "k_proj", "v_proj", "o_proj"), "-": ("up_proj", "down_proj")}


class _Mixer(nn.Module):
    def __init__(self, kind: str) -> None:
        super().__init__()
        for name in _KINDS[kind]:
            setattr(self, name, nn.Linear(1, 1, bias=False))
        self.gate = nn.Linear(1, 1)  # not a reported projection: must stay untouched


class _Layer(nn.Module):
    def __init__(self, kind: str) -> None:
        super().__init__()
        self.mixer = _Mixer(kind)


class _SyntheticNemotron(nn.Module):
    def __init__(self, pattern: str = REPORTED_NEMOTRON_H_8B_PATTERN) -> None:
        super().__init__()
        self.config = types.SimpleNamespace(num_hidden_layers=len(pattern), hybrid_override_pattern=pattern)
        self.layers = nn.ModuleList(_Layer(kind) for kind in pattern)
        self.lm_head = nn.Linear(1, 3, bias=False)


def test_reported_conversion_selects_exactly_112_linears_and_an_fp32_head():
    model = _SyntheticNemotron()
    head_weight = model.lm_head.weight
    result = convert_reported_nemotron_h(model)
    assert len(result.fp4_linears) == 112
    assert result.linear_backend == "probe_matched_triton_issue_rz" and result.probe_matched_backend
    assert isinstance(model.lm_head, FP32OutputLinear) and model.lm_head.weight is head_weight
    converted = [m for m in model.modules() if isinstance(m, UE5M3Linear)]
    assert len(converted) == 112 and all(is_reported_quantized_linear(m) for m in converted)
    assert all(m.scale_state is result.scale_state for m in converted)
    assert isinstance(model.layers[0].mixer.gate, nn.Linear) and not isinstance(model.layers[0].mixer.gate, UE5M3Linear)
    assert model._ue5m3_reported_conversion["fp4_linear_count"] == 112
    assert model.layers[45].mixer.down_proj.module_name == "layers.45.mixer.down_proj"
    assert reported_projection("layers.7.mixer.q_proj") == (7, "q_proj")
    assert reported_projection("layers.0.mixer.q_proj") is None
    assert model.lm_head(torch.ones(2, 1, dtype=torch.bfloat16)).dtype is torch.float32


def test_reported_conversion_rejects_other_architectures():
    with pytest.raises(NemotronHSelectionError, match="52 layers"):
        convert_reported_nemotron_h(_SyntheticNemotron("M-M-"))
    wrong = _SyntheticNemotron()
    wrong.config.hybrid_override_pattern = "M" * 52
    with pytest.raises(NemotronHSelectionError, match="hybrid_override_pattern"):
        convert_reported_nemotron_h(wrong)


def test_trainer_hook_begins_one_step_per_optimizer_step():
    model = _SyntheticNemotron()
    state = convert_reported_nemotron_h(model).scale_state

    class FakeTrainer:
        def __init__(self) -> None:
            self.model_parts = [model]
            self.step = 0
            self.micro_batches = 0

        def train_step(self, micro_batches: int) -> None:
            self.micro_batches += micro_batches

    install_trainer_step_hook(FakeTrainer)
    install_trainer_step_hook(FakeTrainer)  # idempotent
    trainer = FakeTrainer()
    for step in (1, 2, 3):
        trainer.step = step
        trainer.train_step(4)  # four gradient-accumulation micro-batches, one logical step
        assert state.step == step
    assert state.report()["begin_step_calls"] == 3 and trainer.micro_batches == 12
    with pytest.raises(RuntimeError, match="out of order"):
        begin_training_step([model], 3)
    assert begin_training_step([nn.Linear(1, 1)], 1) == 0  # models without FP4 linears: no-op
    # a cold resume far into training simply continues from the trainer's step
    resumed = _SyntheticNemotron()
    resumed_state = convert_reported_nemotron_h(resumed).scale_state
    assert begin_training_step([resumed], 27501) == 1 and resumed_state.step == 27501
