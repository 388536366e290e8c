"""Host-side logic that needs no GPU: recipe, roles and overrides, the D=50 sample-and-hold
state (with an injected sampler: the real one is a device kernel), distributed amax
synchronisation (monkeypatched process group and real gloo ranks), conversion, and the
fail-closed behaviour on CPU tensors.  Mirrors the reference's tests/test_recipe.py,
tests/test_training_scaling.py, tests/test_conversion.py and tests/test_exact_linear.py:81-95."""

from __future__ import annotations

import pytest
import torch
import torch.distributed as dist

from ue5m3_fp4.formats import RoundingMode, normalize_rounding
from ue5m3_fp4.nn import LinearBackend, UE5M3Linear, convert_linear_modules, exclude_lm_head, select_all_linears
from ue5m3_fp4.recipe import OperandRole, UE5M3Recipe
from ue5m3_fp4.scaling import training as training_module
from ue5m3_fp4.scaling.training import TrainingScaleState, sample_global_amax


@pytest.fixture()
def host_sampler(monkeypatch):
    """Replace the device reduction by a host stand-in so the lifecycle can be driven on CPU."""

    monkeypatch.setattr(training_module, "_local_amax", lambda t: t.detach().float().abs().amax())


def test_rounding_and_role_aliases():
    assert normalize_rounding("TiesToEven") is RoundingMode.TIES_TO_EVEN
    assert normalize_rounding("TTE") is RoundingMode.TIES_TO_EVEN
    assert normalize_rounding("StochasticFast") is RoundingMode.STOCHASTIC_8BIT_MIDPOINT
    assert normalize_rounding("stochastic-8bit-midpoint") is RoundingMode.STOCHASTIC_8BIT_MIDPOINT
    with pytest.raises(ValueError, match="unknown rounding mode"):
        normalize_rounding("ideal_stochastic")
    recipe = UE5M3Recipe.proposed()
    assert recipe.normalize_role("dY") is OperandRole.UPSTREAM_GRADIENT
    assert recipe.normalize_role("x") is OperandRole.ACTIVATION
    with pytest.raises(ValueError, match="unknown operand role"):
        recipe.normalize_role("bias")


def test_proposed_recipe_roundings_and_targets():
    recipe = UE5M3Recipe.proposed()
    assert (recipe.block_size, recipe.delayed_scale_interval, recipe.scale_target) == (16, 50, 448.0)
    assert recipe.rounding_for("activation") is RoundingMode.TIES_TO_EVEN
    assert recipe.rounding_for("weight") is RoundingMode.TIES_TO_EVEN
    assert recipe.rounding_for("upstream_gradient") is RoundingMode.STOCHASTIC_8BIT_MIDPOINT
    assert recipe.rounding_for("wgrad_dy") is RoundingMode.STOCHASTIC_8BIT_MIDPOINT
    # The 2048 target applies only to wgrad dY of mixer.down_proj in layers 44..51.
    assert recipe.scale_target_for("wgrad_upstream_gradient", "layers.45.mixer.down_proj") == 2048.0
    assert recipe.scale_target_for("upstream_gradient", "layers.45.mixer.down_proj") == 448.0
    assert recipe.scale_target_for("wgrad_upstream_gradient", "layers.43.mixer.down_proj") == 448.0
    assert recipe.scale_target_for("wgrad_upstream_gradient", "layers.45.mixer.up_proj") == 448.0
    assert recipe.scale_target_for("wgrad_upstream_gradient", "model.layers.51.mixer.down_proj") == 2048.0


def test_recipe_dict_round_trip_and_strictness(tmp_path):
    recipe = UE5M3Recipe.proposed()
    data = recipe.to_dict()
    assert UE5M3Recipe.from_dict(data) == recipe
    with pytest.raises(ValueError, match="invalid recipe keys"):
        UE5M3Recipe.from_dict({**data, "extra": 1})
    with pytest.raises(ValueError, match="ties-to-even"):
        UE5M3Recipe.from_dict({**data, "scale_rounding": "StochasticFast"})
    import yaml

    path = tmp_path / "recipe.yaml"
    path.write_text(yaml.safe_dump(data))
    assert UE5M3Recipe.from_yaml(path) == recipe
    assert UE5M3Recipe.transformer_engine_settings().randomized_hadamard_transform


def test_reference_requires_begin_step_and_increasing_steps(host_sampler):
    state = TrainingScaleState(UE5M3Recipe.proposed())
    with pytest.raises(RuntimeError, match="begin_step"):
        state.reference("activation", "m", torch.ones(4))
    with pytest.raises(ValueError, match="positive"):
        state.begin_step(0)
    state.begin_step(1)
    with pytest.raises(ValueError, match="strictly"):
        state.begin_step(1)


def test_d50_is_sample_and_hold_not_a_window_maximum(host_sampler):
    state = TrainingScaleState(UE5M3Recipe.proposed())
    seen = {}
    for step in range(1, 52):
        state.begin_step(step)
        tensor = {1: torch.tensor([1.0, -3.0]), 51: torch.tensor([1.0, -2.0])}.get(step, torch.tensor([100.0 * step]))
        seen[step] = state.reference("activation", "layers.0.mixer.in_proj", tensor)
    assert [seen[s].item() for s in (1, 2, 50, 51)] == [3.0, 3.0, 3.0, 2.0]
    entry = state.report()["entries"][0]
    assert (entry["last_refresh_step"], entry["refreshes"], entry["reuses"]) == (51, 2, 49)
    assert state.state_dict() == {}


def test_non_finite_samples_stop_the_run_at_the_next_step(host_sampler):
    """The finite check of a sampled amax is deferred: no host read at sampling time, one for
    all samples of a step when the next step begins (or on verify_samples / report)."""

    state = TrainingScaleState(UE5M3Recipe.proposed())
    state.begin_step(1)
    assert state.reference("activation", "a", torch.tensor([2.0])).item() == 2.0
    bad = state.reference("upstream_gradient", "a", torch.tensor([1.0, float("nan")]))
    assert torch.isnan(bad)  # handed out as sampled
    with pytest.raises(ValueError, match=r"non-finite values \(upstream_gradient:a\)"):
        state.begin_step(2)
    state.begin_step(2)  # the offending samples were reported once
    state.reference("weight", "b", torch.tensor([float("inf")]))
    with pytest.raises(ValueError, match="weight:b"):
        state.verify_samples()


def test_weights_are_sampled_together_before_the_forward_pass(monkeypatch, host_sampler):
    calls = []

    def fake_all_reduce(tensor, op=None):
        calls.append((tuple(tensor.shape), op))
        tensor.mul_(2.0)  # stands for a larger value on another rank

    monkeypatch.setattr(dist, "is_initialized", lambda: True)
    monkeypatch.setattr(dist, "get_world_size", lambda: 4)
    monkeypatch.setattr(dist, "get_backend", lambda: "gloo")
    monkeypatch.setattr(dist, "all_reduce", fake_all_reduce)
    state = TrainingScaleState(UE5M3Recipe.proposed())
    with pytest.raises(RuntimeError, match="begin_step"):
        state.sample_weights([("a", torch.ones(2))])
    state.begin_step(1)
    weights = [(f"layers.{i}.mixer.up_proj", torch.full((3, 3), float(i + 1))) for i in range(5)]
    assert state.sample_weights(weights) == 5
    assert calls == [((5,), dist.ReduceOp.MAX)]  # one collective for the five weights
    calls.clear()
    # the linears' own lookups now find the values held: no sampling, no collective
    assert state.reference("weight", "layers.3.mixer.up_proj", torch.zeros(3, 3)).item() == 8.0
    assert calls == [] and state.sample_weights(weights) == 0
    state.begin_step(51)
    assert state.sample_weights(weights[:2]) == 2 and calls == [((2,), dist.ReduceOp.MAX)]
    entries = {e["module_name"]: e for e in state.report()["entries"]}
    assert entries["layers.0.mixer.up_proj"]["refreshes"] == 2 and entries["layers.4.mixer.up_proj"]["refreshes"] == 1


def test_keys_are_per_role_and_module_and_cadence_starts_at_first_use(host_sampler):
    state = TrainingScaleState(UE5M3Recipe.proposed())
    state.begin_step(7)
    assert state.reference("x", "a", torch.tensor([2.0])).item() == 2.0
    assert state.reference("w", "a", torch.tensor([3.0])).item() == 3.0
    assert state.reference("x", "b", torch.tensor([4.0])).item() == 4.0
    assert state.reference("activation", "a", torch.tensor([99.0])).item() == 2.0
    state.begin_step(56)
    assert state.reference("x", "a", torch.tensor([56.0])).item() == 2.0
    state.begin_step(57)
    assert state.reference("x", "a", torch.tensor([57.0])).item() == 57.0
    returned = state.reference("x", "a", torch.tensor([1.0]))
    returned.zero_()  # callers get a clone
    assert state.reference("x", "a", torch.tensor([1.0])).item() == 57.0
    assert state.clear_runtime() == 3 and state.step is None


def test_sampling_has_no_cpu_path():
    state = TrainingScaleState(UE5M3Recipe.proposed())
    state.begin_step(1)
    with pytest.raises(RuntimeError, match="no CPU path"):
        state.reference("activation", "m", torch.ones(4))
    with pytest.raises(ValueError, match="empty"):
        sample_global_amax(torch.ones(0), label="x")
    with pytest.raises(TypeError, match="floating-point"):
        sample_global_amax(torch.ones(2, dtype=torch.int32), label="x")


def test_global_amax_uses_a_max_collective(monkeypatch, host_sampler):
    calls = []

    def fake_all_reduce(tensor, op=None):
        calls.append(op)
        tensor.fill_(11.0)

    monkeypatch.setattr(dist, "is_initialized", lambda: True)
    monkeypatch.setattr(dist, "get_world_size", lambda: 2)
    monkeypatch.setattr(dist, "get_backend", lambda: "gloo")
    monkeypatch.setattr(dist, "all_reduce", fake_all_reduce)
    assert sample_global_amax(torch.tensor([3.0]), label="t").item() == 11.0
    assert calls == [dist.ReduceOp.MAX]
    monkeypatch.setattr(dist, "get_backend", lambda: "nccl")
    with pytest.raises(RuntimeError, match="NCCL"):
        sample_global_amax(torch.tensor([3.0]), label="t")
    monkeypatch.setattr(dist, "get_world_size", lambda: 1)
    calls.clear()
    assert sample_global_amax(torch.tensor([3.0]), label="t").item() == 3.0
    assert calls == []


def test_conversion_keeps_parameters_and_rejects_ambiguity():
    model = torch.nn.Sequential()
    model.add_module("body", torch.nn.Linear(8, 8, bias=False))
    model.add_module("lm_head", torch.nn.Linear(8, 4))
    weight = model.body.weight
    with pytest.raises(ValueError, match="selector is required"):
        convert_linear_modules(model)
    records = convert_linear_modules(model, selector=exclude_lm_head, backend="probe_matched")
    assert [r.module_name for r in records] == ["body"]
    assert isinstance(model.body, UE5M3Linear) and model.body.weight is weight
    assert model.body.backend is LinearBackend.PROBE_MATCHED_TRITON
    assert model.body.backend.value == "probe_matched_triton_issue_rz"
    assert isinstance(model.lm_head, torch.nn.Linear) and not isinstance(model.lm_head, UE5M3Linear)
    shared = torch.nn.Linear(4, 4)
    tied = torch.nn.ModuleDict({"a": shared, "b": shared})
    with pytest.raises(ValueError, match="Aliased"):
        convert_linear_modules(tied, selector=select_all_linears)
    with pytest.raises(ValueError, match="model root"):
        convert_linear_modules(torch.nn.Linear(2, 2), selector=select_all_linears)


def test_product_plan_of_converted_linears():
    """plan_fp4_products: the three GEMM shapes of every converted linear for a token count,
    whether their operands qualify for the packed one-launch quantizers, and the recomputation
    workspace they ask for (host arithmetic only)."""

    from ue5m3_fp4.nn import ConversionRecord, plan_fp4_products

    records = (ConversionRecord("layers.1.mixer.up_proj", 4096, 21504, False),
               ConversionRecord("layers.2.mixer.odd", 100, 64, True))
    plans = plan_fp4_products(records, tokens=8192)
    assert [(p.product, p.m, p.n, p.k) for p in plans[:3]] == [
        ("forward", 8192, 21504, 4096), ("data_gradient", 8192, 4096, 21504), ("weight_gradient", 21504, 4096, 8192)]
    assert all(p.packed_operands for p in plans[:3])
    assert [p.weight_in_one_launch for p in plans[:3]] == [True, True, False]
    assert plans[2].workspace_bytes == (2 * 4096 + 21504 + 4096) * 8192 * 2
    assert [p.packed_operands for p in plans[3:]] == [False, True, True]   # K = 100 is not a multiple of 64
    assert not any(p.weight_in_one_launch for p in plans[3:])
    with pytest.raises(ValueError, match="tokens"):
        plan_fp4_products(records, tokens=0)


def test_linear_fails_closed_on_cpu_and_reports_contract_strings():
    layer = UE5M3Linear(64, 32, bias=False, backend="probe_matched", dtype=torch.bfloat16)
    layer.scale_state.begin_step(1)
    with pytest.raises(RuntimeError, match="requires CUDA operands"):
        layer(torch.ones(4, 64, dtype=torch.bfloat16))
    report = layer.fp4_inference_scaling_report()
    assert report["format"]["gemm_output_model"] == "encoded_operand_k64_issue_rz_bf16_gemm_final_snap_1_over_1024"
    assert report["format"]["native_hardware"] is False
    assert report["format"]["linear_backend"] == "probe_matched_triton_issue_rz"
    with pytest.raises(ValueError, match="Expected input width"):
        layer(torch.ones(4, 63, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="unknown UE5M3 linear backend"):
        UE5M3Linear(4, 4, backend="fastest")


def test_packed_tensor_file_round_trip_on_the_host(tmp_path):
    """The storable packed form (codes + UE5M3 scale bytes + metadata): written and read back
    bit for bit, with the tensor amax kept as its exact fp32 bit pattern; malformed files are
    refused."""

    from ue5m3_fp4.packed import PackedFP4Tensor

    g = torch.Generator().manual_seed(0)
    for rows, cols, block, blocking in ((5, 40, 16, "row"), (70, 96, 32, "2d")):
        scale_rows = rows if blocking == "row" else (rows + block - 1) // block
        packed = PackedFP4Tensor(
            torch.randint(0, 256, (rows, (cols + 1) // 2), generator=g, dtype=torch.int32).to(torch.uint8),
            torch.randint(1, 0xF8, (scale_rows, (cols + block - 1) // block), generator=g, dtype=torch.int32).to(torch.uint8),
            rows, cols, block, blocking, tensor_amax=float(torch.tensor(0.1, dtype=torch.float32)), scale_target=448.0,
            name="layers.3.mixer.down_proj")
        path = tmp_path / f"{blocking}.ue5m3"
        packed.save(path)
        back = PackedFP4Tensor.load(path)
        assert torch.equal(back.codes, packed.codes) and torch.equal(back.scales, packed.scales)
        assert (back.rows, back.cols, back.block_size, back.blocking, back.name) == (rows, cols, block, blocking, packed.name)
        assert back.tensor_amax == packed.tensor_amax and back.scale_target == 448.0
        assert path.stat().st_size < 8 + 8 + 1024 + packed.codes.numel() + packed.scales.numel()
    with pytest.raises(ValueError, match="codes must be"):
        PackedFP4Tensor(torch.zeros(3, 3, dtype=torch.uint8), torch.zeros(3, 1, dtype=torch.uint8), 3, 16, 16, "row", 1.0, 448.0)
    (tmp_path / "bad").write_bytes(b"not a packed tensor at all")
    with pytest.raises(ValueError, match="not a packed"):
        PackedFP4Tensor.load(tmp_path / "bad")
    data = path.read_bytes()
    (tmp_path / "short").write_bytes(data[:-10])
    with pytest.raises(ValueError, match="truncated"):
        PackedFP4Tensor.load(tmp_path / "short")
    with pytest.raises(RuntimeError, match="no CPU path"):
        back.gemm_operand()
