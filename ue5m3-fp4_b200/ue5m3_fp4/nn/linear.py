"""``UE5M3Linear``: an ``nn.Linear`` whose three GEMMs run the probe-matched FP4 model
on the sm_100a kernels.

Public surface of the reference's ``nn/linear.py``: backend names and aliases
(linear.py:43-73), ``UE5M3Linear`` with ``from_float`` (linear.py:423-521), the forward
reference resolution (linear.py:544-599), the nine post-load inference lifecycle methods
(linear.py:624-768) and the module report (linear.py:770-849).  The autograd function
restates linear.py:290-420: which operand takes which role, rounding, target and block
geometry, and that dgrad and wgrad share one held dY amax but draw separate random bits.

Differences from the reference's data flow (same numbers, fewer passes): operands are
quantized straight from their bf16/fp32 storage into encoded bf16 with the reduction axis
contiguous (no fp32 copies, no transposed copies), and snap, alpha, bias and the bf16
cast are fused into the GEMM epilogue.
"""

from __future__ import annotations

from enum import StrEnum
from typing import Any

import torch

from ue5m3_fp4.formats import RoundingMode
from ue5m3_fp4.recipe import UE5M3Recipe
from ue5m3_fp4.scaling.training import TrainingScaleState, sample_global_amax

_ACTIVATION_MODES = ("current_tensor", "training_replay", "calibrated_frozen")


class LinearBackend(StrEnum):
    """Numerical backend names; the strings are part of reports and conversion metadata."""

    PORTABLE = "portable_decoded_torch_reference"
    PROBE_MATCHED_TRITON = "probe_matched_triton_issue_rz"
    TRITON_QUANT_TORCH = "triton_quantized_torch_fp32"


_BACKEND_ALIASES = {
    "portable": LinearBackend.PORTABLE,
    "probe_matched": LinearBackend.PROBE_MATCHED_TRITON,
    "triton": LinearBackend.PROBE_MATCHED_TRITON,
    "torch_control": LinearBackend.TRITON_QUANT_TORCH,
    **{item.value: item for item in LinearBackend},
}


def normalize_linear_backend(value: str | LinearBackend) -> LinearBackend:
    if isinstance(value, LinearBackend):
        return value
    if not isinstance(value, str):
        raise TypeError("backend must be a string or LinearBackend")
    found = _BACKEND_ALIASES.get(value.strip().lower())
    if found is None:
        choices = ", ".join(item.value for item in LinearBackend)
        raise ValueError(f"unknown UE5M3 linear backend {value!r}; expected {choices}")
    return found


def _finite_amax(tensor: torch.Tensor) -> torch.Tensor:
    return sample_global_amax(tensor, label="UE5M3 operand amax")


def _weight_operands_in_one_launch() -> bool:
    """UE5M3_WEIGHT_BOTH=0 makes backward quantize W^T again (as the reference does) instead of
    taking it from the forward pass's single read of the weight."""

    import os

    return os.environ.get("UE5M3_WEIGHT_BOTH", "1") != "0"


def _save_packed_activations() -> bool:
    """Save the packed weight-gradient operand of X instead of the bf16 activations
    (UE5M3_SAVE_PACKED_ACTIVATIONS=0 keeps the bf16 copy, as the reference does)."""

    import os

    return os.environ.get("UE5M3_SAVE_PACKED_ACTIVATIONS", "1").strip() != "0"


def _draw_bits(reference: torch.Tensor):
    """One uniform byte per element for StochasticFast rounding.  By default the bytes are a
    counter-based stream keyed by two draws from the device generator and computed inside the
    quantizer (no bit tensor is written or read); UE5M3_SR_BITS=tensor materialises a uint8
    tensor with torch.randint instead (the reference draws an int32 tensor, linear.py:371-384)."""

    import os

    from ue5m3_fp4.backends import b200

    if os.environ.get("UE5M3_SR_BITS", "philox").strip().lower() == "tensor":
        return torch.randint(0, 256, reference.shape, dtype=torch.uint8, device=reference.device)
    return b200.PhiloxBits.draw(reference.device)


def _reported_quantized_gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    owner: UE5M3Linear,
    role_a: str,
    role_b: str,
    tensor_reference_a: torch.Tensor,
    tensor_reference_b: torch.Tensor,
    two_dimensional_b: bool,
) -> torch.Tensor:
    """One GEMM on logical ``A[M,K]``, ``B[K,N]`` through the public backend entry points
    (linear.py:221-287 of the reference).  Kept for callers that hold logical operands;
    the autograd function below uses the K-major fast path instead."""

    if not a.is_cuda or not b.is_cuda:
        raise RuntimeError(
            "The probe-matched Triton backend requires CUDA operands; "
            "select backend='portable' explicitly for the CPU reference"
        )
    from ue5m3_fp4.backends.triton import (
        fake_quantize_gemm_operands,
        probe_matched_fp4_gemm,
        triton_available,
    )

    if not triton_available():
        raise RuntimeError("The probe-matched Triton backend was requested but CUDA/Triton is unavailable")
    common = {
        "block_size": owner.recipe.block_size,
        "scale_target_a": owner.recipe.scale_target_for(role_a, owner.module_name),
        "scale_target_b": owner.recipe.scale_target_for(role_b, owner.module_name),
        "tensor_amax_a": tensor_reference_a,
        "tensor_amax_b": tensor_reference_b,
        "rounding_a": owner.recipe.rounding_for(role_a),
        "rounding_b": owner.recipe.rounding_for(role_b),
        "two_dimensional_b": two_dimensional_b,
    }
    a = a.contiguous()
    b = b.contiguous()
    if owner.backend is LinearBackend.PROBE_MATCHED_TRITON:
        return probe_matched_fp4_gemm(a, b, **common, snap_to_1_over_1024=True)
    if owner.backend is LinearBackend.TRITON_QUANT_TORCH:
        encoded_a, encoded_b = fake_quantize_gemm_operands(
            a, b, **common, output_domain="encoded", output_dtype=torch.bfloat16
        )
        with torch.autocast(device_type="cuda", enabled=False):
            encoded_output = torch.mm(encoded_a.float(), encoded_b.float())
        alpha = (tensor_reference_a.float() * tensor_reference_b.float()) / (
            (common["scale_target_a"] * 6.0) * (common["scale_target_b"] * 6.0)
        )
        return encoded_output * alpha
    raise AssertionError(f"backend {owner.backend.value!r} is not a reported CUDA backend")


class _OperandPlan:
    """Role -> (target, rounding) lookups of one module, resolved once per call."""

    def __init__(self, owner: UE5M3Linear) -> None:
        from ue5m3_fp4.backends import b200

        self.recipe = owner.recipe
        self.name = owner.module_name
        self.owner = owner
        self.block = owner.recipe.block_size
        # FP4 tensor cores for the probe-matched backend unless the environment asks for the
        # BF16-issue kernel; the torch control always multiplies encoded bf16 operands.
        probe = owner.backend is LinearBackend.PROBE_MATCHED_TRITON
        self.path = b200.gemm_path() if probe else "bf16"

    def target(self, role: str) -> float:
        return self.recipe.scale_target_for(role, self.name)

    def rounding(self, role: str) -> RoundingMode:
        return self.recipe.rounding_for(role)


def _encode_k_major(
    tensor: torch.Tensor,
    *,
    plan: _OperandPlan,
    role: str,
    reference: torch.Tensor,
    reduce_over_rows: bool,
    two_dimensional: bool,
    bits: torch.Tensor | None = None,
    hadamard: bool = False,
):
    """Quantize ``tensor`` [R, C] into a GEMM operand with the reduction axis contiguous
    ([R, C] when the GEMM reduces over C, [C, R] when it reduces over R; the quantizer writes
    the transpose itself).  On the FP4 path the operand is packed codes + tensor-core scale
    factors, on the BF16-issue path the encoded values ``p*s`` as bf16."""

    from ue5m3_fp4.backends import b200

    rounding = plan.rounding(role)
    if rounding is RoundingMode.STOCHASTIC_8BIT_MIDPOINT and bits is None:
        bits = _draw_bits(tensor)
    if two_dimensional:
        blocking = b200.BLOCK_2D
    else:
        blocking = b200.BLOCK_COL if reduce_over_rows else b200.BLOCK_ROW
    if plan.path == "fp4":
        # one binade of headroom: a held amax may lag the data between refreshes
        operand = b200.quantize_fp4_operand(
            tensor, block_size=plan.block, blocking=blocking, transposed=reduce_over_rows,
            tensor_amax=reference.reshape(1), scale_target=plan.target(role), rounding=rounding,
            random_bits=bits, shift_headroom=1, hadamard=hadamard,
        )
        histograms = plan.owner.__dict__.get("_scale_histograms")
        if histograms is not None:  # opt-in diagnostics: block-scale code counts per operand role
            key = f"{plan.recipe.normalize_role(role).value}{'_along_rows' if reduce_over_rows else ''}"
            histograms[key] = b200.scale_byte_histogram(operand, block_size=plan.block, two_dimensional=two_dimensional,
                                                        out=histograms.get(key))
        return operand
    if hadamard:
        raise NotImplementedError(
            "the Hadamard-transformed weight-gradient operands exist on the FP4 tensor-core path only "
            "(UE5M3_GEMM_PATH=fp4)"
        )
    packed = b200.quantize_packed(
        tensor,
        block_size=plan.block,
        blocking=blocking,
        tensor_amax=reference.reshape(1),
        scale_target=plan.target(role),
        rounding=rounding,
        random_bits=bits,
        packed=False,
        packed_t=False,
        fake_domain="encoded",
        fake_dtype=torch.bfloat16,
        fake=not reduce_over_rows,
        fake_t=reduce_over_rows,
    )
    return packed.fake_t if reduce_over_rows else packed.fake


def _gemm(
    a_enc,
    bt_enc,
    *,
    owner: UE5M3Linear,
    reference_a: torch.Tensor,
    reference_b: torch.Tensor,
    target_a: float,
    target_b: float,
    bias: torch.Tensor | None,
    out_dtype: torch.dtype,
) -> torch.Tensor:
    from ue5m3_fp4.backends import b200

    # alpha = fl(fl(amax_a*amax_b) / ((Ta*6)*(Tb*6))) is formed inside the GEMM epilogue from the
    # two held amaxes (no launch of its own)
    alpha = b200.EpilogueAlpha.of(reference_a, reference_b, target_a, target_b)
    if isinstance(a_enc, b200.Fp4Operand):
        return b200.gemm_fp4_operands(a_enc, bt_enc, snap=True, alpha=alpha, bias=bias, out_dtype=out_dtype)
    if owner.backend is LinearBackend.PROBE_MATCHED_TRITON:
        return b200.gemm_issue_rz(a_enc, bt_enc, snap=True, alpha=alpha, bias=bias, out_dtype=out_dtype)
    # torch control: same encoded operands, library FP32 matrix multiplication
    alpha = b200.encoded_global_alpha(reference_a.reshape(1), reference_b.reshape(1), target_a, target_b)
    with torch.autocast(device_type="cuda", enabled=False):
        out = torch.mm(a_enc.float(), bt_enc.float().t()) * alpha
    if bias is not None:
        out = out + bias.to(torch.float32)
    return out.to(out_dtype)


class _ProbeMatchedUE5M3LinearFunction(torch.autograd.Function):
    """Y = X W^T, dX = dY W, dW = dY^T X under the probe-matched FP4 model."""

    @staticmethod
    def forward(ctx: Any, inputs: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
                owner: UE5M3Linear) -> torch.Tensor:
        if owner._inference["active"] and torch.is_grad_enabled():
            raise RuntimeError("Post-load FP4 inference is forward-only")
        if not inputs.is_cuda or not weight.is_cuda:
            raise RuntimeError(
                "The probe-matched Triton backend requires CUDA operands; "
                "select backend='portable' explicitly for the CPU reference"
            )
        if inputs.dtype is not torch.bfloat16:
            raise TypeError(
                "The probe-matched reported path requires BF16 activations at the linear boundary"
            )
        if weight.dtype not in {torch.bfloat16, torch.float32}:
            raise TypeError("The probe-matched path requires BF16 or FP32 master weights")
        plan = _OperandPlan(owner)
        x = inputs.reshape(-1, inputs.shape[-1]).contiguous()
        w = weight.detach().contiguous()
        activation_reference = owner._forward_reference("activation", x)
        weight_reference = owner._forward_reference("weight", w)
        two_d = owner.recipe.two_dimensional_weights
        rht = owner.recipe.randomized_hadamard_transform and not owner._inference["active"]
        activation_rht_reference = None
        if rht:
            # The forward GEMM stays untransformed; this current amax belongs to the transformed
            # X^T that the weight-gradient GEMM reads (linear.py:316-324 of the reference).
            from ue5m3_fp4.backends import b200

            if plan.path != "fp4":
                raise NotImplementedError(
                    "the Hadamard-transformed weight-gradient comparator exists on the FP4 tensor-core "
                    "path only (UE5M3_GEMM_PATH=fp4)"
                )
            activation_rht_reference = _finite_amax(b200.hadamard_amax_transposed(x))
        x_enc = _encode_k_major(x, plan=plan, role="activation", reference=activation_reference,
                                reduce_over_rows=False, two_dimensional=False)
        w_enc = owner._packed_frozen_weight(weight, weight_reference, plan) if owner._inference["active"] else None
        wt_enc = None
        if (w_enc is None and two_d and plan.path == "fp4" and ctx.needs_input_grad[0] and _weight_operands_in_one_launch()
                and not owner._inference["active"] and owner.__dict__.get("_scale_histograms") is None
                and plan.rounding("weight") is RoundingMode.TIES_TO_EVEN):
            # The data-gradient GEMM of this step reads W^T with the same B x B block scales: both
            # orientations leave one launch that reads W once (the reference quantizes the weight
            # again in backward, linear.py:359-363).  W^T travels to backward as saved tensors.
            from ue5m3_fp4.backends import b200

            both = b200.quantize_fp4_operand_both(w, block_size=plan.block, tensor_amax=weight_reference.reshape(1),
                                                  scale_target=plan.target("weight"), shift_headroom=1)
            if both is not None:
                w_enc, wt_enc = both
        if w_enc is None:
            w_enc = _encode_k_major(w, plan=plan, role="weight", reference=weight_reference,
                                    reduce_over_rows=False, two_dimensional=two_d)
            if owner._inference["active"]:
                owner._remember_packed_frozen_weight(weight, weight_reference, plan, w_enc)
        output = _gemm(
            x_enc, w_enc, owner=owner, reference_a=activation_reference, reference_b=weight_reference,
            target_a=plan.target("activation"), target_b=plan.target("weight"),
            bias=None if bias is None else bias.detach().contiguous(), out_dtype=torch.bfloat16,
        )
        ctx.owner = owner
        ctx.has_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        ctx.activation_reference = activation_reference.detach()
        ctx.weight_reference = weight_reference.detach()
        ctx.activation_rht_reference = None if activation_rht_reference is None else activation_rht_reference.detach()
        ctx.input_shape = inputs.shape
        ctx.packed_activation = None
        if (plan.path == "fp4" and _save_packed_activations() and ctx.needs_input_grad[1]
                and owner.__dict__.get("_grad_mode_at_call", True)
                and x.shape[0] % 64 == 0):  # the weight-gradient GEMM reduces over the tokens
            # The weight-gradient GEMM reads X^T blocked along the tokens with the SAME held
            # reference, so its packed operand (0.5625 byte per element) can be made now and
            # saved instead of the bf16 activations (2 bytes per element; the packed form also keeps
            # the unmodified UE5M3 scale bytes, 0.625 byte per element in all); the result is the
            # operand the backward would have built (the reference re-quantizes a saved bf16
            # copy, linear.py:346,385-398).
            xt = _encode_k_major(x, plan=plan, role="activation",
                                 reference=activation_rht_reference if rht else activation_reference,
                                 reduce_over_rows=True, two_dimensional=False, hadamard=rht)
            ctx.packed_activation = (xt.shift, xt.rows, xt.k)
            saved = [weight, xt.codes, xt.scale_factors, xt.raw_scale_factors, xt.record]
        else:
            saved = [weight, inputs]
        ctx.packed_weight_t = None
        if wt_enc is not None:
            ctx.packed_weight_t = (wt_enc.shift, wt_enc.rows, wt_enc.k, len(saved))
            saved += [wt_enc.codes, wt_enc.scale_factors, wt_enc.raw_scale_factors, wt_enc.record]
        ctx.save_for_backward(*saved)
        return output.reshape(*inputs.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx: Any, grad_output: torch.Tensor):
        owner: UE5M3Linear = ctx.owner
        if owner._inference["active"]:
            raise RuntimeError("Backward is forbidden after FP4 inference is configured")
        from ue5m3_fp4.backends import b200

        plan = _OperandPlan(owner)
        two_d = owner.recipe.two_dimensional_weights
        saved = ctx.saved_tensors
        weight = saved[0]
        if ctx.packed_activation is not None:
            xt_codes, xt_scales, xt_raw_scales, xt_record = saved[1:5]
            shift, rows, k = ctx.packed_activation
            xt_saved = b200.Fp4Operand(xt_codes, xt_scales, shift, rows, k, xt_raw_scales, xt_record)
            x = None
        else:
            inputs = saved[1]
            xt_saved = None
            x = inputs.to(torch.bfloat16).reshape(-1, inputs.shape[-1]).contiguous()
        wt_saved = None
        if ctx.packed_weight_t is not None:
            shift, rows, k, first = ctx.packed_weight_t
            wt_saved = b200.Fp4Operand(saved[first], saved[first + 1], shift, rows, k, saved[first + 2], saved[first + 3])
        dy = grad_output.to(torch.bfloat16).reshape(-1, grad_output.shape[-1]).contiguous()
        w = weight.detach().contiguous()

        # One held dY amax serves both backward GEMMs; the random bits are drawn per GEMM.
        dy_reference = owner.scale_state.reference("upstream_gradient", owner.module_name, dy)

        # dX[M,K] = dY[M,N] . W[N,K]: reduce over N; W is read with N contiguous -> transpose
        dy_enc = _encode_k_major(dy, plan=plan, role="upstream_gradient", reference=dy_reference,
                                 reduce_over_rows=False, two_dimensional=False)
        wt_enc = wt_saved if wt_saved is not None else _encode_k_major(
            w, plan=plan, role="weight", reference=ctx.weight_reference, reduce_over_rows=True, two_dimensional=two_d)
        grad_input = _gemm(
            dy_enc, wt_enc, owner=owner, reference_a=dy_reference, reference_b=ctx.weight_reference,
            target_a=plan.target("upstream_gradient"), target_b=plan.target("weight"),
            bias=None, out_dtype=torch.bfloat16,
        )
        del dy_enc, wt_enc

        # dW[N,K] = dY^T[N,M] . X[M,K]: reduce over the tokens M; both operands are
        # blocked along M and written transposed, so M is contiguous.
        rht = owner.recipe.randomized_hadamard_transform
        wgrad_dy_reference, wgrad_x_reference = dy_reference, ctx.activation_reference
        if rht:
            # The only transformed GEMM of the TE-settings comparator: both operands carry the
            # fixed-sign B=16 Hadamard transform along the tokens, dY^T with the current amax of
            # the transformed tensor, X^T with the one sampled in forward (linear.py:389-400).
            if ctx.activation_rht_reference is None:
                raise RuntimeError("missing saved transformed-activation amax for RHT wgrad")
            wgrad_dy_reference = _finite_amax(b200.hadamard_amax_transposed(dy))
            wgrad_x_reference = ctx.activation_rht_reference
        dyt_enc = _encode_k_major(dy, plan=plan, role="wgrad_upstream_gradient", reference=wgrad_dy_reference,
                                  reduce_over_rows=True, two_dimensional=False, hadamard=rht)
        xt_enc = xt_saved if xt_saved is not None else _encode_k_major(
            x, plan=plan, role="activation", reference=wgrad_x_reference,
            reduce_over_rows=True, two_dimensional=False, hadamard=rht)
        grad_weight = _gemm(
            dyt_enc, xt_enc, owner=owner, reference_a=wgrad_dy_reference, reference_b=wgrad_x_reference,
            target_a=plan.target("wgrad_upstream_gradient"), target_b=plan.target("activation"),
            bias=None, out_dtype=weight.dtype,
        )
        grad_bias = None
        if ctx.has_bias:
            # fp32 accumulation straight from the bf16 rows: no fp32 copy of dY is materialised
            grad_bias = dy.sum(dim=0, dtype=torch.float32).to(ctx.bias_dtype)
        return grad_input.reshape(ctx.input_shape), grad_weight, grad_bias, None


def _fresh_inference_state(generation: int, cleared: bool, entries: int) -> dict[str, Any]:
    return {
        "active": False,
        "generation": generation,
        "phase": "inactive",
        "activation_mode": None,
        "frozen_weights": {},
        "frozen_activations": {},
        "activation_calibration_max": 0.0,
        "activation_calibration_count": 0,
        "training_replay_logical_step": 0,
        "training_replay_last_consumed_step": 0,
        "training_replay_cache": 0.0,
        "training_replay_last_refresh_step": 0,
        "training_replay_refresh_trace": [],
        "legacy_training_state_cleared": {
            "runtime_cache_cleared": cleared,
            "delayed_amax_entries": entries,
            "training_cache_inherited": False,
        },
        "counters": {
            "resets": generation,
            "weight_calibrations": 0,
            "weight_frozen_resolutions": 0,
            "activation_current_resolutions": 0,
            "activation_calibration_resolutions": 0,
            "activation_frozen_resolutions": 0,
            "activation_replay_refreshes": 0,
            "activation_replay_reuses": 0,
        },
    }


class UE5M3Linear(torch.nn.Module):
    """``nn.Linear``-compatible FP4 linear.  Call ``scale_state.begin_step(step)`` once per
    training step; for quantized evaluation drive the inference lifecycle through
    :class:`ue5m3_fp4.scaling.FP4InferenceScalingController` after loading the checkpoint."""

    def __init__(
        self,
        in_features: int,
        out_features: int,
        bias: bool = True,
        *,
        recipe: UE5M3Recipe | None = None,
        scale_state: TrainingScaleState | None = None,
        backend: str | LinearBackend = LinearBackend.PROBE_MATCHED_TRITON,
        module_name: str = "linear",
        device: torch.device | str | None = None,
        dtype: torch.dtype | None = None,
        _initialize_parameters: bool = True,
    ) -> None:
        super().__init__()
        if in_features <= 0 or out_features <= 0:
            raise ValueError("in_features and out_features must be positive")
        if not module_name:
            raise ValueError("module_name must be non-empty")
        self.in_features = int(in_features)
        self.out_features = int(out_features)
        self.recipe = recipe or UE5M3Recipe.proposed()
        if scale_state is not None and scale_state.recipe != self.recipe:
            raise ValueError("scale_state.recipe must match the linear recipe")
        self.scale_state = scale_state or TrainingScaleState(self.recipe)
        self.backend = normalize_linear_backend(backend)
        if self.recipe.randomized_hadamard_transform:
            if self.recipe != UE5M3Recipe.transformer_engine_settings():
                raise ValueError(
                    "the public RHT implementation accepts only the reported "
                    "UE5M3 Transformer-Engine-settings recipe"
                )
            if self.backend is not LinearBackend.PROBE_MATCHED_TRITON:
                raise ValueError(
                    "the reported UE5M3 RHT comparator requires the probe-matched Triton backend"
                )
        self.module_name = module_name
        factory = {"device": device, "dtype": dtype}
        self.weight = torch.nn.Parameter(torch.empty(out_features, in_features, **factory))
        if bias:
            self.bias = torch.nn.Parameter(torch.empty(out_features, **factory))
        else:
            self.register_parameter("bias", None)
        if _initialize_parameters:
            self.reset_parameters()
        self._inference_generation = 0
        self._inference: dict[str, Any] = {}
        self.reset_fp4_inference_scaling(clear_training_state=False)

    def reset_parameters(self) -> None:
        torch.nn.init.kaiming_uniform_(self.weight, a=5**0.5)
        if self.bias is not None:
            fan_in = self.weight.shape[1]
            bound = 1 / fan_in**0.5 if fan_in > 0 else 0
            torch.nn.init.uniform_(self.bias, -bound, bound)

    @classmethod
    def from_float(cls, module: torch.nn.Linear, *, recipe: UE5M3Recipe, scale_state: TrainingScaleState,
                   backend: str | LinearBackend = LinearBackend.PROBE_MATCHED_TRITON,
                   module_name: str) -> UE5M3Linear:
        if not isinstance(module, torch.nn.Linear):
            raise TypeError("from_float expects torch.nn.Linear")
        converted = cls(
            module.in_features, module.out_features, bias=module.bias is not None, recipe=recipe,
            scale_state=scale_state, backend=backend, module_name=module_name, device="meta",
            dtype=module.weight.dtype, _initialize_parameters=False,
        )
        # The very same Parameter objects: optimizer references, tying and meta
        # parameters survive the swap.
        converted.weight = module.weight
        if module.bias is not None:
            converted.bias = module.bias
        return converted

    @staticmethod
    def _reference_tensor(value: float, tensor: torch.Tensor) -> torch.Tensor:
        return torch.tensor(value, device=tensor.device, dtype=torch.float32)

    # After checkpoint load the weight and its amax are frozen, so the forward operand of W
    # (packed codes + scale atoms, or encoded values on the BF16-issue path) is built once and
    # reused until the parameter is written again; the reference re-quantizes the weight in
    # every forward (linear.py:549-554,710-718).
    def _packed_weight_key(self, weight: torch.Tensor, reference: torch.Tensor, plan) -> tuple:
        return (weight.data_ptr(), weight._version, tuple(weight.shape), weight.dtype,
                self._inference["frozen_weights"].get("forward.w"), plan.path, plan.block,
                self.recipe.two_dimensional_weights)

    def capture_scale_histograms(self, enable: bool = True) -> None:
        """Start (or stop and drop) counting the UE5M3 block-scale bytes of every operand this
        layer quantizes on the FP4 path: ``scale_histograms()`` then maps an operand role
        (``activation``, ``weight``, ``upstream_gradient``, and with ``_along_rows`` appended the
        operands blocked along the tokens for the weight-gradient product) to 256 counters.  The
        counts come from the scale bytes the quantizers write anyway; the tensors are not read
        again.  Device-side form of reproduce/scale_target/capture_scale_target_histograms.py of
        the reference."""

        self.__dict__["_scale_histograms"] = {} if enable else None

    def scale_histograms(self) -> dict[str, torch.Tensor]:
        return dict(self.__dict__.get("_scale_histograms") or {})

    def export_packed_weight(self, path) -> None:
        """Write this layer's weight, quantized with its FROZEN amax, as a packed FP4 tensor file
        (``ue5m3_fp4.packed.PackedFP4Tensor``): what a quantized-evaluation run needs of the
        weight, at 0.5625 byte per element.  Requires the post-load lifecycle to have frozen the
        weight scale."""

        from ue5m3_fp4.packed import PackedFP4Tensor

        frozen = self._inference["frozen_weights"].get("forward.w") if self._inference["active"] else None
        if frozen is None:
            raise RuntimeError("Weight amax has not been frozen after checkpoint load")
        PackedFP4Tensor.quantize(
            self.weight.detach(), block_size=self.recipe.block_size, two_dimensional=self.recipe.two_dimensional_weights,
            tensor_amax=float(frozen), scale_target=self.recipe.scale_target_for("weight", self.module_name),
            name=self.module_name).save(path)

    def load_packed_weight(self, path) -> None:
        """Install a packed weight written by ``export_packed_weight`` as this layer's forward
        operand, so that no forward pass quantizes the weight.  The file must describe this
        layer's weight under this layer's recipe and frozen amax; the operand is dropped again
        as soon as the parameter is written to."""

        from ue5m3_fp4.packed import PackedFP4Tensor

        plan = _OperandPlan(self)
        if plan.path != "fp4":
            raise RuntimeError("packed weights feed the FP4 tensor-core path (UE5M3_GEMM_PATH=fp4)")
        frozen = self._inference["frozen_weights"].get("forward.w") if self._inference["active"] else None
        if frozen is None:
            raise RuntimeError("Weight amax has not been frozen after checkpoint load")
        packed = PackedFP4Tensor.load(path, self.weight.device)
        expect = (self.out_features, self.in_features, self.recipe.block_size,
                  "2d" if self.recipe.two_dimensional_weights else "row",
                  self.recipe.scale_target_for("weight", self.module_name))
        found = (packed.rows, packed.cols, packed.block_size, packed.blocking, packed.scale_target)
        if found != expect:
            raise ValueError(f"packed weight {found} does not match this layer {expect}")
        if packed.tensor_amax != float(torch.tensor(float(frozen), dtype=torch.float32)):
            raise ValueError("packed weight was quantized with another tensor amax than the frozen one")
        reference = self._reference_tensor(float(frozen), self.weight)
        self._remember_packed_frozen_weight(self.weight, reference, plan, packed.gemm_operand(shift_headroom=1))

    def _packed_frozen_weight(self, weight: torch.Tensor, reference: torch.Tensor, plan):
        cached = self.__dict__.get("_packed_weight_cache")
        if cached is not None and cached[0] == self._packed_weight_key(weight, reference, plan):
            return cached[1]
        return None

    def _remember_packed_frozen_weight(self, weight: torch.Tensor, reference: torch.Tensor, plan, operand) -> None:
        self.__dict__["_packed_weight_cache"] = (self._packed_weight_key(weight, reference, plan), operand)

    def _forward_reference(self, role: str, tensor: torch.Tensor) -> torch.Tensor:
        state = self._inference
        if not state["active"]:
            return self.scale_state.reference(role, self.module_name, tensor)
        counters = state["counters"]
        if role == "weight":
            value = state["frozen_weights"].get("forward.w")
            if value is None:
                raise RuntimeError("Weight amax has not been frozen after checkpoint load")
            counters["weight_frozen_resolutions"] += 1
            return self._reference_tensor(value, tensor)
        if role != "activation":
            raise RuntimeError(f"Inference does not resolve role {role!r}")
        phase, mode = state["phase"], state["activation_mode"]
        if phase == "activation_calibration":
            current = float(_finite_amax(tensor).item())
            state["activation_calibration_max"] = max(state["activation_calibration_max"], current)
            state["activation_calibration_count"] += 1
            counters["activation_calibration_resolutions"] += 1
            return self._reference_tensor(current, tensor)
        if phase != "measuring":
            raise RuntimeError(f"FP4 inference forward is not allowed in phase {phase!r}")
        if mode == "current_tensor":
            counters["activation_current_resolutions"] += 1
            return self._reference_tensor(float(_finite_amax(tensor).item()), tensor)
        if mode == "calibrated_frozen":
            value = state["frozen_activations"].get("forward.x")
            if value is None:
                raise RuntimeError("Activation amax has not been frozen")
            counters["activation_frozen_resolutions"] += 1
            return self._reference_tensor(value, tensor)
        if mode == "training_replay":
            step = state["training_replay_logical_step"]
            if step <= 0:
                raise RuntimeError("Advance the replay work unit before each forward")
            if state["training_replay_last_consumed_step"] == step:
                raise RuntimeError(f"Replay step {step} was consumed twice")
            last = state["training_replay_last_refresh_step"]
            if last == 0 or step - last >= 50:
                current = float(_finite_amax(tensor).item())
                state["training_replay_cache"] = current
                state["training_replay_last_refresh_step"] = step
                state["training_replay_refresh_trace"].append({"logical_step": step, "amax": current})
                counters["activation_replay_refreshes"] += 1
            else:
                counters["activation_replay_reuses"] += 1
            state["training_replay_last_consumed_step"] = step
            return self._reference_tensor(state["training_replay_cache"], tensor)
        raise RuntimeError(f"Unsupported inference activation mode {mode!r}")

    def forward(self, inputs: torch.Tensor) -> torch.Tensor:
        if inputs.shape[-1] != self.in_features:
            raise ValueError(f"Expected input width {self.in_features}, got {inputs.shape[-1]}")
        if self._inference["active"] and torch.is_grad_enabled():
            raise RuntimeError(
                "Post-load FP4 inference requires torch.no_grad() or torch.inference_mode()"
            )
        if self.backend is LinearBackend.PORTABLE:
            raise RuntimeError(
                "the portable decoded-torch reference is a CPU model and is not part of the "
                "B200 package; use backend='probe_matched' (CUDA, sm_100a)"
            )
        self.__dict__["_grad_mode_at_call"] = torch.is_grad_enabled()  # forward() itself runs without grad mode
        return _ProbeMatchedUE5M3LinearFunction.apply(inputs, self.weight, self.bias, self)

    # ---- post-load inference lifecycle (module protocol of scaling/inference.py:36-46) ----
    def reset_fp4_inference_scaling(self, *, clear_training_state: bool = True) -> dict[str, Any]:
        if type(clear_training_state) is not bool:
            raise TypeError("clear_training_state must be bool")
        cleared = self.scale_state.clear_runtime() if clear_training_state else 0
        self._inference_generation += 1
        self._inference = _fresh_inference_state(self._inference_generation, clear_training_state, cleared)
        self.__dict__.pop("_packed_weight_cache", None)
        return {
            "generation": self._inference_generation,
            "legacy_training_state_cleared": dict(self._inference["legacy_training_state_cleared"]),
        }

    def configure_fp4_inference_scaling(self, activation_mode: str) -> None:
        if self.training:
            raise RuntimeError("Call model.eval() before configuring FP4 inference")
        if (
            torch.distributed.is_available()
            and torch.distributed.is_initialized()
            and torch.distributed.get_world_size() > 1
        ):
            raise RuntimeError("The deterministic FP4 inference scaling protocol requires one process")
        stochastic = {
            name: mode.value
            for name, mode in (
                ("activation_rounding", self.recipe.activation_rounding),
                ("weight_rounding", self.recipe.weight_rounding),
                ("scale_rounding", self.recipe.scale_rounding),
            )
            if mode is RoundingMode.STOCHASTIC_8BIT_MIDPOINT
        }
        if stochastic:
            details = ", ".join(f"{name}={mode}" for name, mode in sorted(stochastic.items()))
            raise ValueError(f"Deterministic FP4 inference rejects stochastic forward rounding: {details}")
        if activation_mode not in _ACTIVATION_MODES:
            raise ValueError(f"Unknown FP4 inference mode {activation_mode!r}")
        if activation_mode == "training_replay" and self.recipe.delayed_scale_interval != 50:
            raise ValueError(
                "training_replay implements the recorded D=50 protocol and "
                "requires delayed_scale_interval=50"
            )
        state = self._inference
        if state["active"]:
            raise RuntimeError("FP4 inference scaling was configured twice")
        state.update(active=True, activation_mode=activation_mode, phase="configured")

    def calibrate_and_freeze_fp4_inference_weight_scale(self) -> dict[str, Any]:
        state = self._inference
        if state["phase"] != "configured":
            raise RuntimeError("Weight calibration requires configured inference")
        value = float(_finite_amax(self.weight).item())
        state["frozen_weights"]["forward.w"] = value
        state["counters"]["weight_calibrations"] += 1
        state["phase"] = "weights_frozen"
        return {"key": "forward.w", "amax": value, "device": self.weight.device.type}

    def begin_fp4_inference_activation_calibration(self) -> None:
        state = self._inference
        if state["activation_mode"] != "calibrated_frozen":
            raise RuntimeError("Activation calibration requires calibrated_frozen mode")
        if state["phase"] != "weights_frozen":
            raise RuntimeError("Freeze weights before activation calibration")
        state.update(activation_calibration_max=0.0, activation_calibration_count=0,
                     phase="activation_calibration")

    def freeze_fp4_inference_activation_scales(self) -> dict[str, Any]:
        state = self._inference
        if state["phase"] != "activation_calibration":
            raise RuntimeError("No activation calibration is active")
        if state["activation_calibration_count"] <= 0:
            raise RuntimeError("No activation operands were observed")
        value, count = state["activation_calibration_max"], state["activation_calibration_count"]
        state["frozen_activations"]["forward.x"] = value
        state["phase"] = "activations_frozen"
        return {"forward.x": {"amax": value, "observations": count}}

    def begin_fp4_inference_measurement(self) -> None:
        state = self._inference
        expected = "activations_frozen" if state["activation_mode"] == "calibrated_frozen" else "weights_frozen"
        if state["phase"] != expected:
            raise RuntimeError(f"Measurement requires phase {expected!r}, got {state['phase']!r}")
        state["phase"] = "measuring"

    def advance_fp4_inference_training_replay_step(self, logical_step: int) -> None:
        state = self._inference
        if state["activation_mode"] != "training_replay":
            raise RuntimeError("Replay advancement requires training_replay mode")
        expected = state["training_replay_logical_step"] + 1
        if logical_step != expected:
            raise RuntimeError(f"Expected replay step {expected}, got {logical_step}")
        state["training_replay_logical_step"] = logical_step

    def reset_fp4_inference_measurement_counters(self) -> None:
        counters = self._inference["counters"]
        for name in counters:
            if name not in {"resets", "weight_calibrations"}:
                counters[name] = 0

    def fp4_inference_scaling_report(self) -> dict[str, Any]:
        state = self._inference
        probe_matched = self.backend is LinearBackend.PROBE_MATCHED_TRITON
        torch_control = self.backend is LinearBackend.TRITON_QUANT_TORCH
        policy: dict[str, Any] = {
            "input_dtype": "bfloat16" if probe_matched else "float32",
            "device_type": self.weight.device.type,
            "torch_float32_matmul_precision": None,
            "cuda_matmul_fp32_precision": None,
            "cuda_matmul_allow_tf32": None,
        }
        if self.weight.device.type == "cuda":
            if hasattr(torch.backends.cuda.matmul, "fp32_precision"):
                policy["cuda_matmul_fp32_precision"] = str(torch.backends.cuda.matmul.fp32_precision)
            else:
                policy["torch_float32_matmul_precision"] = torch.get_float32_matmul_precision()
                policy["cuda_matmul_allow_tf32"] = bool(torch.backends.cuda.matmul.allow_tf32)
        if probe_matched:
            output_model = "encoded_operand_k64_issue_rz_bf16_gemm_final_snap_1_over_1024"
        elif torch_control:
            output_model = "encoded_operand_torch_fp32_matmul"
        else:
            output_model = "decoded_operand_torch_matmul"
        rht = bool(self.recipe.randomized_hadamard_transform)
        return {
            "schema": "ue5m3_fp4_inference_module_scaling_v1",
            "active": state["active"],
            "generation": state["generation"],
            "phase": state["phase"],
            "activation_mode": state["activation_mode"],
            "frozen_global_amax": {
                "weights": dict(state["frozen_weights"]),
                "activations": dict(state["frozen_activations"]),
            },
            "activation_calibration_counts": {"forward.x": state["activation_calibration_count"]},
            "counters": dict(state["counters"]),
            "legacy_training_state_cleared": dict(state["legacy_training_state_cleared"]),
            "rounding_modes": {
                "round_mode_activations": self.recipe.activation_rounding,
                "round_mode_weights": self.recipe.weight_rounding,
            },
            "training_replay": {
                "interval": self.recipe.delayed_scale_interval,
                "logical_step": state["training_replay_logical_step"],
                "last_consumed_step": state["training_replay_last_consumed_step"],
                "cache": {"forward.x": state["training_replay_cache"]},
                "last_refresh_steps": {"forward.x": state["training_replay_last_refresh_step"]},
                "refresh_trace": {"forward.x": list(state["training_replay_refresh_trace"])},
            },
            "format": {
                "payload": self.recipe.payload_format.name,
                "block_size": self.recipe.block_size,
                "scale_type": self.recipe.scale_format.name,
                "scale_max_activations": self.recipe.scale_target_for("activation", self.module_name),
                "scale_max_weights": self.recipe.scale_target_for("weight", self.module_name),
                "gemm_output_model": output_model,
                "torch_matmul_policy": policy,
                "native_hardware": False,
                "encode_centric": probe_matched or torch_control,
                "use_encoded_gemm": probe_matched or torch_control,
                "linear_backend": self.backend.value,
                "randomized_hadamard_transform": {
                    "forward_gemm": False,
                    "data_gradient_gemm": False,
                    "weight_gradient_operands": rht,
                    "block_size": 16 if rht else None,
                },
            },
        }


__all__ = ["LinearBackend", "UE5M3Linear", "normalize_linear_backend"]
