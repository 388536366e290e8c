"""Numerical controls of one UE5M3 FP4 training recipe.

Same public surface and semantics as the reference's ``recipe.py``: operand roles
and aliases (recipe.py:25-64), the structured scale-target override for
``mixer.down_proj`` layers (recipe.py:67-138) and the strict recipe dataclass with
its dict/YAML forms (recipe.py:157-407).
"""

from __future__ import annotations

import math
import re
from collections.abc import Mapping
from dataclasses import dataclass, fields
from enum import StrEnum
from pathlib import Path
from typing import Any

from ue5m3_fp4.formats import E2M1, UE5M3, FloatFormat, RoundingMode, normalize_rounding


class OperandRole(StrEnum):
    """Operands that keep their own delayed-amax state."""

    ACTIVATION = "activation"
    WEIGHT = "weight"
    UPSTREAM_GRADIENT = "upstream_gradient"
    WGRAD_UPSTREAM_GRADIENT = "wgrad_upstream_gradient"


_ROLE_NAMES = {
    OperandRole.ACTIVATION: ("activation", "activations", "x", "input"),
    OperandRole.WEIGHT: ("weight", "weights", "w"),
    OperandRole.UPSTREAM_GRADIENT: ("upstream_gradient", "upstream_gradients", "dy", "d_y"),
    OperandRole.WGRAD_UPSTREAM_GRADIENT: (
        "wgrad_upstream_gradient",
        "wgrad_dy",
        "weight_gradient_upstream_gradient",
    ),
}
_ROLE_LOOKUP = {name: role for role, names in _ROLE_NAMES.items() for name in names}


def normalize_role(role: str | OperandRole) -> OperandRole:
    if isinstance(role, OperandRole):
        return role
    if not isinstance(role, str):
        raise TypeError("role must be a string or OperandRole")
    found = _ROLE_LOOKUP.get(role.strip().replace("-", "_").lower())
    if found is None:
        choices = ", ".join(item.value for item in OperandRole)
        raise ValueError(f"unknown operand role {role!r}; expected {choices}")
    return found


_DOWN_PROJ = re.compile(r"(?:^|\.)layers\.(?P<layer>\d+)\.mixer\.down_proj(?:$|\.)")


def _positive_finite(value: Any) -> bool:
    return type(value) in (int, float) and math.isfinite(float(value)) and value > 0


@dataclass(frozen=True, slots=True)
class ScaleTargetOverride:
    """Scale target for one operand role inside a range of ``mixer.down_proj`` layers."""

    role: OperandRole
    module_kind: str
    layer_start: int
    layer_end: int
    scale_target: float

    _KEYS = ("role", "module_kind", "layer_start", "layer_end", "scale_target")

    def __post_init__(self) -> None:
        object.__setattr__(self, "role", normalize_role(self.role))
        if self.module_kind != "mixer.down_proj":
            raise ValueError("the public recipe supports module_kind='mixer.down_proj'")
        if type(self.layer_start) is not int or type(self.layer_end) is not int:
            raise TypeError("layer bounds must be integers")
        if self.layer_start < 0 or self.layer_end < self.layer_start:
            raise ValueError("invalid layer bounds")
        if not _positive_finite(self.scale_target):
            raise ValueError("override scale_target must be a finite positive number")

    def matches(self, role: str | OperandRole, module_name: str) -> bool:
        if normalize_role(role) is not self.role:
            return False
        if not isinstance(module_name, str):
            raise TypeError("module_name must be a string")
        found = _DOWN_PROJ.search(module_name)
        return found is not None and self.layer_start <= int(found.group("layer")) <= self.layer_end

    def to_dict(self) -> dict[str, Any]:
        return {
            "role": self.role.value,
            "module_kind": self.module_kind,
            "layer_start": self.layer_start,
            "layer_end": self.layer_end,
            "scale_target": float(self.scale_target),
        }

    @classmethod
    def from_dict(cls, value: Mapping[str, Any]) -> ScaleTargetOverride:
        if not isinstance(value, Mapping):
            raise TypeError("each scale-target override must be a mapping")
        expected = set(cls._KEYS)
        unknown, missing = set(value) - expected, expected - set(value)
        if unknown or missing:
            raise ValueError(f"invalid override keys; missing={sorted(missing)}, unknown={sorted(unknown)}")
        return cls(**{key: value[key] for key in cls._KEYS})


def _format_field(value: Any, *, expected: FloatFormat) -> FloatFormat:
    if isinstance(value, FloatFormat):
        result = value
    elif isinstance(value, str):
        known = {E2M1.name.lower(): E2M1, UE5M3.name.lower(): UE5M3}
        if value.strip().lower() not in known:
            raise ValueError(f"unknown floating-point format {value!r}")
        result = known[value.strip().lower()]
    else:
        raise TypeError("format fields must be format names or FloatFormat instances")
    if result != expected:
        raise ValueError(f"this recipe requires {expected.name}, got {result.name}")
    return result


_ROUNDING_FIELDS = ("activation_rounding", "weight_rounding", "upstream_gradient_rounding", "scale_rounding")


@dataclass(frozen=True, slots=True)
class UE5M3Recipe:
    """Complete numerical controls; delayed scaling is periodic sample-and-hold."""

    name: str
    block_size: int
    payload_format: FloatFormat
    scale_format: FloatFormat
    scale_target: float
    delayed_scale_interval: int
    activation_rounding: RoundingMode
    weight_rounding: RoundingMode
    upstream_gradient_rounding: RoundingMode
    scale_rounding: RoundingMode
    two_dimensional_weights: bool
    randomized_hadamard_transform: bool
    scale_target_overrides: tuple[ScaleTargetOverride, ...] = ()

    def __post_init__(self) -> None:
        put = lambda key, value: object.__setattr__(self, key, value)  # noqa: E731
        if not isinstance(self.name, str) or not self.name.strip():
            raise ValueError("recipe name must be a non-empty string")
        if type(self.block_size) is not int or self.block_size <= 0:
            raise ValueError("block_size must be a positive integer")
        put("payload_format", _format_field(self.payload_format, expected=E2M1))
        put("scale_format", _format_field(self.scale_format, expected=UE5M3))
        if not _positive_finite(self.scale_target):
            raise ValueError("scale_target must be a finite positive number")
        if type(self.delayed_scale_interval) is not int or self.delayed_scale_interval <= 0:
            raise ValueError("delayed_scale_interval must be a positive integer")
        for key in _ROUNDING_FIELDS:
            put(key, normalize_rounding(getattr(self, key)))
        if self.scale_rounding is not RoundingMode.TIES_TO_EVEN:
            raise ValueError("UE5M3 block scales use ties-to-even rounding")
        if type(self.two_dimensional_weights) is not bool:
            raise TypeError("two_dimensional_weights must be bool")
        if type(self.randomized_hadamard_transform) is not bool:
            raise TypeError("randomized_hadamard_transform must be bool")
        put("scale_target_overrides", tuple(self.scale_target_overrides))
        if any(not isinstance(item, ScaleTargetOverride) for item in self.scale_target_overrides):
            raise TypeError("scale_target_overrides must contain ScaleTargetOverride values")
        if self.randomized_hadamard_transform and self._te_signature() != _TE_SIGNATURE:
            raise ValueError(
                "this portable recipe does not implement RHT for arbitrary "
                "controls; use UE5M3Recipe.transformer_engine_settings()"
            )

    def _te_signature(self) -> tuple:
        return (
            self.block_size,
            float(self.scale_target),
            self.delayed_scale_interval,
            self.activation_rounding,
            self.weight_rounding,
            self.upstream_gradient_rounding,
            self.two_dimensional_weights,
            self.scale_target_overrides,
        )

    @classmethod
    def proposed(cls) -> UE5M3Recipe:
        """The proposed B=16, D=50 periodic-refresh recipe (recipe.py:239-265)."""

        return cls(
            name="proposed_ue5m3_b16_d50",
            block_size=16,
            payload_format=E2M1,
            scale_format=UE5M3,
            scale_target=448.0,
            delayed_scale_interval=50,
            activation_rounding=RoundingMode.TIES_TO_EVEN,
            weight_rounding=RoundingMode.TIES_TO_EVEN,
            upstream_gradient_rounding=RoundingMode.STOCHASTIC_8BIT_MIDPOINT,
            scale_rounding=RoundingMode.TIES_TO_EVEN,
            two_dimensional_weights=True,
            randomized_hadamard_transform=False,
            scale_target_overrides=(
                ScaleTargetOverride(OperandRole.WGRAD_UPSTREAM_GRADIENT, "mixer.down_proj", 44, 51, 2_048.0),
            ),
        )

    @classmethod
    def transformer_engine_settings(cls) -> UE5M3Recipe:
        """The UE5M3 comparator with TE-style controls, D=1 and the wgrad Hadamard transform
        (recipe.py:267-293).  Kept for configuration parity; its transform kernels are not built."""

        return cls(
            name="ue5m3_b16_transformer_engine_settings_d1",
            block_size=16,
            payload_format=E2M1,
            scale_format=UE5M3,
            scale_target=448.0,
            delayed_scale_interval=1,
            activation_rounding=RoundingMode.TIES_TO_EVEN,
            weight_rounding=RoundingMode.TIES_TO_EVEN,
            upstream_gradient_rounding=RoundingMode.STOCHASTIC_8BIT_MIDPOINT,
            scale_rounding=RoundingMode.TIES_TO_EVEN,
            two_dimensional_weights=True,
            randomized_hadamard_transform=True,
            scale_target_overrides=(),
        )

    @staticmethod
    def normalize_role(role: str | OperandRole) -> OperandRole:
        return normalize_role(role)

    def rounding_for(self, role: str | OperandRole) -> RoundingMode:
        """Payload rounding of a GEMM operand role; both dY roles share one mode."""

        normalized = normalize_role(role)
        if normalized is OperandRole.ACTIVATION:
            return self.activation_rounding
        if normalized is OperandRole.WEIGHT:
            return self.weight_rounding
        return self.upstream_gradient_rounding

    def scale_target_for(self, role: str | OperandRole, module_name: str) -> float:
        """Tensor-scale target of one (role, module): first matching override, else the default."""

        normalized = normalize_role(role)
        if not isinstance(module_name, str):
            raise TypeError("module_name must be a string")
        for override in self.scale_target_overrides:
            if override.matches(normalized, module_name):
                return float(override.scale_target)
        return float(self.scale_target)

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"schema_version": 1}
        for item in fields(self):
            value = getattr(self, item.name)
            if isinstance(value, FloatFormat):
                value = value.name
            elif isinstance(value, RoundingMode):
                value = value.value
            elif item.name == "scale_target":
                value = float(value)
            elif item.name == "scale_target_overrides":
                value = [entry.to_dict() for entry in value]
            out[item.name] = value
        return out

    @classmethod
    def from_dict(cls, value: Mapping[str, Any]) -> UE5M3Recipe:
        if not isinstance(value, Mapping):
            raise TypeError("recipe configuration must be a mapping")
        data = dict(value)
        version = data.pop("schema_version", 1)
        if version != 1:
            raise ValueError(f"unsupported recipe schema_version {version!r}")
        expected = {item.name for item in fields(cls)}
        unknown, missing = set(data) - expected, expected - set(data)
        if unknown or missing:
            raise ValueError(f"invalid recipe keys; missing={sorted(missing)}, unknown={sorted(unknown)}")
        data["scale_target_overrides"] = tuple(
            ScaleTargetOverride.from_dict(entry) for entry in data["scale_target_overrides"]
        )
        return cls(**data)

    @classmethod
    def from_yaml(cls, path: str | Path) -> UE5M3Recipe:
        try:
            import yaml
        except ImportError as error:  # pragma: no cover
            raise RuntimeError("PyYAML is required to load recipe files") from error
        with Path(path).open("r", encoding="utf-8") as handle:
            return cls.from_dict(yaml.safe_load(handle))


_TE_SIGNATURE = (
    16,
    448.0,
    1,
    RoundingMode.TIES_TO_EVEN,
    RoundingMode.TIES_TO_EVEN,
    RoundingMode.STOCHASTIC_8BIT_MIDPOINT,
    True,
    (),
)

__all__ = ["OperandRole", "ScaleTargetOverride", "UE5M3Recipe", "normalize_role"]
