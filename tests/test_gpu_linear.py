"""GPU tests of UE5M3Linear: forward equals the public composition, the three GEMMs take
the roles / roundings / targets / block geometry of the reference (tests/test_exact_linear.py:
98-139,298-330), backward matches the oracle with explicit random bits, and the D=50
lifecycle refreshes at steps 1, 51 and 101 over 120 steps."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from gpu_helpers import bf16_round, oracle_quantize, random_bits, to_np
from oracle import ue5m3_oracle as o

pytestmark = pytest.mark.gpu


def _layer(in_f, out_f, *, bias, name="layers.0.mixer.up_proj", recipe=None, dtype=torch.bfloat16, seed=0):
    from ue5m3_fp4.nn import UE5M3Linear

    torch.manual_seed(seed)
    layer = UE5M3Linear(in_f, out_f, bias=bias, recipe=recipe, backend="probe_matched", module_name=name,
                        device="cuda", dtype=dtype)
    with torch.no_grad():
        layer.weight.copy_(0.02 * torch.randn(out_f, in_f))
    return layer


def test_forward_equals_public_composition(gemm_path):
    from ue5m3_fp4.backends.triton import probe_matched_fp4_gemm

    layer = _layer(256, 192, bias=True)
    layer.scale_state.begin_step(1)
    x = torch.randn(4, 32, 256, device="cuda").to(torch.bfloat16)
    y = layer(x)
    flat = x.reshape(-1, 256)
    ref = probe_matched_fp4_gemm(
        flat, layer.weight.detach().float().t().contiguous(), block_size=16,
        tensor_amax_a=flat.float().abs().amax(), tensor_amax_b=layer.weight.detach().float().abs().amax(),
        two_dimensional_b=True,
    )
    ref = (ref + layer.bias.detach().float()).to(torch.bfloat16).reshape(4, 32, 192)
    assert y.dtype is torch.bfloat16 and torch.equal(y, ref)


@pytest.mark.parametrize("name,block", [("layers.45.mixer.down_proj", 16), ("layers.3.mixer.in_proj", 32)])
def test_backward_matches_oracle_with_explicit_bits(monkeypatch, gemm_path, name, block):
    import ue5m3_fp4.nn.linear as linear_module
    from ue5m3_fp4.recipe import UE5M3Recipe

    recipe = UE5M3Recipe.proposed()
    if block == 32:
        recipe = UE5M3Recipe.from_dict({**recipe.to_dict(), "block_size": 32, "name": "b32"})
    tokens, in_f, out_f = 128, 192, 128  # every reduction axis is a multiple of 64
    layer = _layer(in_f, out_f, bias=True, name=name, recipe=recipe, dtype=torch.float32, seed=3)
    layer.scale_state.begin_step(1)
    draws = []

    def fixed_bits(reference):
        bits = random_bits(reference.shape, seed=100 + len(draws), dtype=torch.uint8).to(reference.device)
        draws.append(bits)
        return bits

    monkeypatch.setattr(linear_module, "_draw_bits", fixed_bits)
    g = torch.Generator().manual_seed(9)
    x = torch.relu(torch.randn(tokens, in_f, generator=g)).square().to(torch.bfloat16).cuda().requires_grad_(True)
    dy = (1e-4 * torch.randn(tokens, out_f, generator=g)).to(torch.bfloat16).cuda()
    y = layer(x)
    y.backward(dy)
    torch.cuda.synchronize()
    from ue5m3_fp4.backends import b200

    b200.check_gemm_status(x.device)  # bounded waits and the FP4 scale window
    assert len(draws) == 2  # separate draws for dgrad and wgrad

    w = layer.weight.detach().float().cpu()
    xh, dyh = x.detach().float().cpu(), dy.float().cpu()
    ax, aw, ady = float(xh.abs().max()), float(w.abs().max()), float(dyh.abs().max())
    t_wdy = recipe.scale_target_for("wgrad_upstream_gradient", name)
    assert t_wdy == (2048.0 if "down_proj" in name and block == 16 else 448.0) or block == 32
    qx = oracle_quantize(xh, block=block, blocking=o.BLOCK_ROW, amax=ax)
    qw = oracle_quantize(w, block=block, blocking=o.BLOCK_2D, amax=aw)
    yo = o.gemm_issue_rz(qx["encoded"], qw["encoded"], snap=True, alpha_value=o.alpha(np.float32(ax), np.float32(aw), 448.0, 448.0))
    yo = bf16_round(yo + to_np(layer.bias.detach()))
    assert np.array_equal(to_np(y), yo)
    # dgrad: dY rows (stochastic, first draw) x W^T with the same 2-D tiles
    qdy = oracle_quantize(dyh, block=block, blocking=o.BLOCK_ROW, amax=ady, sr=True, bits=draws[0])
    dxo = o.gemm_issue_rz(qdy["encoded"], np.ascontiguousarray(qw["encoded"].T), snap=True,
                          alpha_value=o.alpha(np.float32(ady), np.float32(aw), 448.0, 448.0))
    assert np.array_equal(to_np(x.grad), bf16_round(dxo))
    # wgrad: dY^T and X^T, both blocked along the tokens; second draw; T override on dY only
    qdyt = oracle_quantize(dyh, block=block, blocking=o.BLOCK_COL, amax=ady, target=t_wdy, sr=True, bits=draws[1])
    qxt = oracle_quantize(xh, block=block, blocking=o.BLOCK_COL, amax=ax)
    dwo = o.gemm_issue_rz(np.ascontiguousarray(qdyt["encoded"].T), np.ascontiguousarray(qxt["encoded"].T), snap=True,
                          alpha_value=o.alpha(np.float32(ady), np.float32(ax), t_wdy, 448.0))
    assert layer.weight.grad.dtype is torch.float32
    assert np.array_equal(to_np(layer.weight.grad), dwo)
    assert np.array_equal(to_np(layer.bias.grad), dyh.numpy().sum(0, dtype=np.float32)) or torch.allclose(
        layer.bias.grad.cpu(), dyh.sum(0), rtol=1e-6, atol=0)
    keys = {(e["role"], e["module_name"]) for e in layer.scale_state.report()["entries"]}
    assert keys == {("activation", name), ("weight", name), ("upstream_gradient", name)}


def test_delayed_scaling_refreshes_at_1_51_101_over_120_steps():
    layer = _layer(128, 64, bias=False, name="layers.45.mixer.down_proj")
    refreshed = []
    import ue5m3_fp4.scaling.training as training

    original = layer.scale_state._sample_amax

    def counting(tensor, name="sample"):
        refreshed.append(layer.scale_state.step)
        return original(tensor, name)

    layer.scale_state._sample_amax = counting
    g = torch.Generator(device="cuda").manual_seed(1)
    for step in range(1, 121):
        layer.scale_state.begin_step(step)
        x = (torch.randn(64, 128, device="cuda", generator=g) * (1 + step % 7)).to(torch.bfloat16).requires_grad_(True)
        layer(x).backward(torch.randn(64, 64, device="cuda", generator=g).to(torch.bfloat16) * 1e-4)
        layer.weight.grad = None
    assert sorted(set(refreshed)) == [1, 51, 101]
    assert len(refreshed) == 9  # activation, weight, upstream gradient at each refresh
    for entry in layer.scale_state.report()["entries"]:
        assert (entry["refreshes"], entry["reuses"], entry["last_refresh_step"]) == (3, 117, 101)


def test_inference_lifecycle_current_tensor_and_frozen():
    from ue5m3_fp4.scaling import FP4InferenceScalingController

    model = torch.nn.Sequential()
    model.add_module("proj", _layer(128, 64, bias=False, name="proj"))
    model.eval()
    x = torch.randn(32, 128, device="cuda").to(torch.bfloat16)
    controller = FP4InferenceScalingController(model, activation_mode="calibrated_frozen",
                                               checkpoint_identity={"name": "synthetic"})
    controller.reset_after_checkpoint_load()
    controller.calibrate_and_freeze_weights()
    controller.begin_activation_calibration({"set": "unit"})
    with torch.no_grad():
        controller.record_activation_calibration_batch(x)
        model(x)
        controller.record_activation_calibration_batch(x * 2)
        model(x * 2)
    frozen = controller.freeze_activation_scales()
    assert frozen["proj"]["forward.x"]["amax"] == (x * 2).float().abs().max().item()
    controller.begin_measurement()
    with pytest.raises(RuntimeError, match="no_grad"):
        model(x)
    with torch.no_grad():
        y = model(x)
    assert y.shape == (32, 64)
    provenance = controller.provenance()
    assert provenance["numeric_path"] == "quantized_ue5m3_fp4_probe_matched_k64_issue_rz"
    assert provenance["native_hardware"] is False
    assert controller.counters()["proj"]["activation_frozen_resolutions"] == 1


def test_inference_lifecycle_training_replay():
    """Post-load inference that replays the D = 50 training cadence: the activation amax is
    sampled at work units 1 and 51 and held in between (nn/linear.py:575-598 of the reference),
    every forward is preceded by one work-unit advancement, and a second forward inside one
    work unit is refused."""

    from ue5m3_fp4.scaling import FP4InferenceScalingController

    model = torch.nn.Sequential()
    model.add_module("proj", _layer(128, 64, bias=False, name="proj"))
    model.eval()
    with pytest.raises(ValueError, match="replay_work_unit"):
        FP4InferenceScalingController(model, activation_mode="training_replay", checkpoint_identity={"name": "synthetic"})
    controller = FP4InferenceScalingController(
        model, activation_mode="training_replay", checkpoint_identity={"name": "synthetic"},
        replay_work_unit={"kind": "fixed_forward_batch", "size": 32})
    controller.reset_after_checkpoint_load()
    controller.calibrate_and_freeze_weights()
    with pytest.raises(ValueError, match="evaluation_order"):
        controller.begin_measurement()
    controller.begin_measurement(evaluation_order={"order": "sequential", "seed": 0})
    g = torch.Generator(device="cuda").manual_seed(3)
    ids = torch.zeros(32, 8, dtype=torch.int64, device="cuda")
    with torch.no_grad():
        with pytest.raises(RuntimeError, match="Advance the replay work unit"):
            model(torch.randn(32, 128, device="cuda", generator=g).to(torch.bfloat16))
        amaxes, outputs = {}, {}
        for unit in range(1, 53):
            x = (torch.randn(32, 128, device="cuda", generator=g) * (1 + unit % 5)).to(torch.bfloat16)
            controller.advance_training_replay_work_unit(ids + unit, effective_token_count=256)
            outputs[unit] = model(x)
            amaxes[unit] = x.float().abs().max().item()
            if unit == 7:
                with pytest.raises(RuntimeError, match="consumed twice"):
                    model(x)
        with pytest.raises(ValueError, match="fixed forward batch"):
            controller.advance_training_replay_work_unit(ids[:5], effective_token_count=40)
    report = model.proj.fp4_inference_scaling_report()["training_replay"]
    assert [entry["logical_step"] for entry in report["refresh_trace"]["forward.x"]] == [1, 51]
    assert [entry["amax"] for entry in report["refresh_trace"]["forward.x"]] == [amaxes[1], amaxes[51]]
    assert report["last_consumed_step"] == 52 and report["cache"]["forward.x"] == amaxes[51]
    counters = controller.counters()["proj"]
    assert counters["activation_replay_refreshes"] == 2 and counters["activation_replay_reuses"] == 50
    assert len(controller.training_replay_work_units) == 52
    # a held step really quantizes with the amax of work unit 1: same input, other reference -> other output
    assert outputs[2].shape == (32, 64) and torch.isfinite(outputs[2].float()).all()


def test_scale_byte_histograms_against_the_oracle(monkeypatch):
    """Block-scale code counts as a by-product of the operand quantizers (read from the scale
    bytes, not from the tensors) equal a numpy count of the oracle's scale codes: forward X of a
    squared-ReLU layer (with all-zero blocks), the 2-D weight tiles, dY, and the two operands
    blocked along the tokens; B = 16 and 32."""

    monkeypatch.setenv("UE5M3_GEMM_PATH", "fp4")
    from ue5m3_fp4.recipe import UE5M3Recipe

    for block in (16, 32):
        recipe = UE5M3Recipe.proposed()
        if block == 32:
            recipe = UE5M3Recipe.from_dict({**recipe.to_dict(), "block_size": 32, "name": "b32"})
        tokens, in_f, out_f = 192, 256, 128
        name = "layers.47.mixer.down_proj"
        layer = _layer(in_f, out_f, bias=False, name=name, recipe=recipe, seed=block)
        layer.capture_scale_histograms()
        layer.scale_state.begin_step(1)
        g = torch.Generator().manual_seed(block)
        x = torch.relu(torch.randn(tokens, in_f, generator=g)).square()
        x[:, 64:64 + block] = 0.0       # all-zero blocks along the features ...
        x[32:64, 7] = 0.0               # ... and along the tokens
        x = x.to(torch.bfloat16).cuda().requires_grad_(True)
        dy = (1e-4 * torch.randn(tokens, out_f, generator=g)).to(torch.bfloat16).cuda()
        layer(x).backward(dy)
        got = {key: value.cpu().numpy() for key, value in layer.scale_histograms().items()}
        assert sorted(got) == ["activation", "activation_along_rows", "upstream_gradient", "weight",
                               "weight_along_rows", "wgrad_upstream_gradient_along_rows"]
        xh, wh, dyh = x.detach().float().cpu(), layer.weight.detach().float().cpu(), dy.float().cpu()
        ax, aw, ady = float(xh.abs().max()), float(wh.abs().max()), float(dyh.abs().max())
        t_wgrad = recipe.scale_target_for("wgrad_upstream_gradient", name)

        def count(tensor, blocking, amax, target=448.0):
            q = oracle_quantize(tensor, block=block, blocking=blocking, amax=amax, target=target)
            codes = q["scale_codes"].astype(np.int64).copy()
            codes[q["block_amax"] == 0] = 0       # bin 0: blocks whose elements are all zero
            return np.bincount(codes.reshape(-1), minlength=256)

        assert np.array_equal(got["activation"], count(xh, o.BLOCK_ROW, ax))
        assert np.array_equal(got["activation_along_rows"], count(xh, o.BLOCK_COL, ax))
        assert np.array_equal(got["weight"], count(wh, o.BLOCK_2D, aw))
        assert np.array_equal(got["weight_along_rows"], count(wh, o.BLOCK_2D, aw))
        assert np.array_equal(got["upstream_gradient"], count(dyh, o.BLOCK_ROW, ady))
        assert np.array_equal(got["wgrad_upstream_gradient_along_rows"], count(dyh, o.BLOCK_COL, ady, t_wgrad))
        assert got["activation"][0] >= tokens and got["activation_along_rows"][0] >= 32 // block
        # a second step accumulates
        layer.scale_state.begin_step(2)
        layer.weight.grad = None
        layer(x).backward(dy)
        assert np.array_equal(layer.scale_histograms()["weight"].cpu().numpy(), 2 * got["weight"])
        layer.capture_scale_histograms(False)
        assert layer.scale_histograms() == {}


def test_packed_weight_file_feeds_the_frozen_inference_path(tmp_path, monkeypatch):
    """export_packed_weight / load_packed_weight: the weight of a frozen layer goes to a packed
    file (0.5625 byte per element) and comes back as the forward operand; outputs are identical
    and the weight is not quantized again."""

    from ue5m3_fp4.backends import b200
    from ue5m3_fp4.packed import PackedFP4Tensor
    from ue5m3_fp4.scaling import FP4InferenceScalingController

    monkeypatch.setenv("UE5M3_GEMM_PATH", "fp4")

    def frozen_model(seed):
        model = torch.nn.Sequential()
        model.add_module("proj", _layer(256, 192, bias=True, name="proj", seed=seed))
        model.eval()
        controller = FP4InferenceScalingController(model, activation_mode="current_tensor",
                                                   checkpoint_identity={"name": "synthetic"})
        controller.reset_after_checkpoint_load()
        controller.calibrate_and_freeze_weights()
        controller.begin_measurement()
        return model

    first = frozen_model(seed=8)
    x = torch.randn(64, 256, device="cuda").to(torch.bfloat16)
    with torch.no_grad():
        expect = first(x)
    path = tmp_path / "proj.ue5m3"
    first.proj.export_packed_weight(path)
    weight = first.proj.weight
    assert path.stat().st_size < weight.numel() * 0.5625 + 1024
    packed = PackedFP4Tensor.load(path, "cuda")
    direct = b200.quantize_packed(weight.detach(), block_size=16, blocking=b200.BLOCK_2D,
                                  tensor_amax=b200.tensor_amax(weight.detach()).reshape(1), packed=True, packed_t=False)
    assert torch.equal(packed.codes, direct.codes) and torch.equal(packed.scales, direct.scales)
    assert torch.equal(packed.dequantize(), b200.dequantize_packed(
        direct.codes, direct.scales, rows=192, cols=256, block_size=16, two_dimensional=True,
        tensor_amax=b200.tensor_amax(weight.detach()).reshape(1)))

    second = frozen_model(seed=8)   # the same weights, loaded "from a checkpoint"
    second.proj.load_packed_weight(path)
    calls = []
    original = b200.quantize_fp4_operand

    def counting(tensor, **kwargs):
        calls.append(tuple(tensor.shape))
        return original(tensor, **kwargs)

    monkeypatch.setattr(b200, "quantize_fp4_operand", counting)
    with torch.no_grad():
        got = second(x)
        again = second(x)
    assert torch.equal(got, expect) and torch.equal(again, expect)
    assert calls == [(64, 256), (64, 256)]  # activations only: the weight came from the file
    other = frozen_model(seed=9)
    with pytest.raises(ValueError, match="another tensor amax"):
        other.proj.load_packed_weight(path)


def test_packed_activation_saving_keeps_gradients_and_shrinks_what_is_saved(monkeypatch):
    """On the FP4 path the forward saves the packed weight-gradient operand of X (codes +
    scale atoms, the raw scale bytes and the small window record) instead of the bf16
    activations: same gradients, bit for bit, and less than a third of the bytes held for
    backward."""

    import ue5m3_fp4.nn.linear as linear_module

    tokens, in_f, out_f = 1024, 2048, 384
    results = {}
    monkeypatch.setenv("UE5M3_WEIGHT_BOTH", "0")   # the weight's second operand is a saved tensor of its own
    for mode in ("1", "0"):
        monkeypatch.setenv("UE5M3_GEMM_PATH", "fp4")
        monkeypatch.setenv("UE5M3_SAVE_PACKED_ACTIVATIONS", mode)
        layer = _layer(in_f, out_f, bias=False, seed=5)
        layer.scale_state.begin_step(1)
        draws = []

        def fixed_bits(reference, draws=draws):
            bits = random_bits(reference.shape, seed=40 + len(draws), dtype=torch.uint8).to(reference.device)
            draws.append(bits)
            return bits

        monkeypatch.setattr(linear_module, "_draw_bits", fixed_bits)
        g = torch.Generator().manual_seed(2)
        x = torch.randn(tokens, in_f, generator=g).to(torch.bfloat16).cuda().requires_grad_(True)
        dy = (1e-3 * torch.randn(tokens, out_f, generator=g)).to(torch.bfloat16).cuda()
        saved = []
        with torch.autograd.graph.saved_tensors_hooks(lambda t: (saved.append(t.numel() * t.element_size()), t)[1],
                                                      lambda t: t):
            y = layer(x)
        y.backward(dy)
        torch.cuda.synchronize()
        results[mode] = (y.detach().clone(), x.grad.clone(), layer.weight.grad.clone(), sum(saved))
    for a, b in zip(results["1"][:3], results["0"][:3]):
        assert torch.equal(a, b)
    weight_bytes = out_f * in_f * 2
    packed_extra = results["1"][3] - weight_bytes
    bf16_extra = results["0"][3] - weight_bytes
    assert bf16_extra == tokens * in_f * 2
    assert packed_extra * 3 < bf16_extra


def test_weight_quantized_once_per_step_keeps_gradients(monkeypatch):
    """By default the forward pass makes both operands of the weight (W for Y = X W^T, W^T for
    dX = dY W) in one launch and hands W^T to backward; with UE5M3_WEIGHT_BOTH=0 backward
    quantizes the weight again as the reference does.  Same outputs and gradients, bit for bit;
    the saved W^T operand costs 0.5625 + 0.0625 byte per weight element until backward has run."""

    import ue5m3_fp4.nn.linear as linear_module

    tokens, in_f, out_f = 256, 320, 192
    results = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("UE5M3_GEMM_PATH", "fp4")
        monkeypatch.setenv("UE5M3_WEIGHT_BOTH", mode)
        layer = _layer(in_f, out_f, bias=True, seed=6)
        layer.scale_state.begin_step(1)
        draws = []

        def fixed_bits(reference, draws=draws):
            bits = random_bits(reference.shape, seed=70 + len(draws), dtype=torch.uint8).to(reference.device)
            draws.append(bits)
            return bits

        monkeypatch.setattr(linear_module, "_draw_bits", fixed_bits)
        g = torch.Generator().manual_seed(4)
        x = torch.randn(tokens, in_f, generator=g).to(torch.bfloat16).cuda().requires_grad_(True)
        dy = (1e-3 * torch.randn(tokens, out_f, generator=g)).to(torch.bfloat16).cuda()
        saved = []
        with torch.autograd.graph.saved_tensors_hooks(lambda t: (saved.append(t.numel() * t.element_size()), t)[1],
                                                      lambda t: t):
            y = layer(x)
        y.backward(dy)
        torch.cuda.synchronize()
        results[mode] = (y.detach().clone(), x.grad.clone(), layer.weight.grad.clone(), layer.bias.grad.clone(), sum(saved))
    for a, b in zip(results["1"][:4], results["0"][:4]):
        assert torch.equal(a, b)
    extra = results["1"][4] - results["0"][4]
    assert out_f * in_f * 0.625 <= extra <= out_f * in_f * 0.625 + 4 * (4 + 4096 + 2 * in_f) + 4096


def test_frozen_weight_operand_is_built_once_in_inference(monkeypatch):
    """After the weight scale is frozen the forward operand of W is cached until the parameter
    is written again; outputs equal those of a layer that quantizes the weight every time."""

    import ue5m3_fp4.nn.linear as linear_module
    from ue5m3_fp4.scaling import FP4InferenceScalingController

    calls = []
    original = linear_module._encode_k_major

    def counting(tensor, **kw):
        calls.append(kw["role"])
        return original(tensor, **kw)

    monkeypatch.setattr(linear_module, "_encode_k_major", counting)
    model = torch.nn.Sequential()
    model.add_module("proj", _layer(256, 128, bias=False, name="proj"))
    model.eval()
    controller = FP4InferenceScalingController(model, activation_mode="current_tensor",
                                               checkpoint_identity={"name": "synthetic"})
    controller.reset_after_checkpoint_load()
    controller.calibrate_and_freeze_weights()
    controller.begin_measurement()
    x = torch.randn(64, 256, device="cuda").to(torch.bfloat16)
    with torch.no_grad():
        y1 = model(x)
        y2 = model(x)
        y3 = model(x * 0.5)
    assert calls.count("weight") == 1 and calls.count("activation") == 3
    assert torch.equal(y1, y2)
    # a fresh layer with the same weights, training-style forward with the same references
    fresh = _layer(256, 128, bias=False, name="proj")
    fresh.scale_state.begin_step(1)
    with torch.no_grad():
        assert torch.equal(fresh(x), y1)
    # writing the parameter invalidates the cached operand
    before = calls.count("weight")
    with torch.no_grad():
        model(x)
        assert calls.count("weight") == before  # still cached
        model.proj.weight.mul_(0.5)
        model(x)
    assert calls.count("weight") == before + 1
    assert y3.shape == (64, 128)


def test_te_settings_comparator_backward_matches_oracle(monkeypatch):
    """UE5M3 with TE settings (D=1, fixed-sign B=16 Hadamard transform on the two weight-gradient
    operands only): forward and data gradient untransformed, weight gradient on the transformed
    dY^T and X^T with the amax of the transformed tensors (nn/linear.py:316-324,389-400)."""

    import ue5m3_fp4.nn.linear as linear_module
    from ue5m3_fp4.backends import b200
    from ue5m3_fp4.recipe import UE5M3Recipe

    monkeypatch.setenv("UE5M3_GEMM_PATH", "fp4")
    recipe = UE5M3Recipe.transformer_engine_settings()
    tokens, in_f, out_f = 128, 192, 128
    name = "layers.7.mixer.up_proj"
    layer = _layer(in_f, out_f, bias=False, name=name, recipe=recipe, dtype=torch.float32, seed=4)
    layer.scale_state.begin_step(1)
    draws = []

    def fixed_bits(reference):
        bits = random_bits(reference.shape, seed=300 + len(draws), dtype=torch.uint8).to(reference.device)
        draws.append(bits)
        return bits

    monkeypatch.setattr(linear_module, "_draw_bits", fixed_bits)
    g = torch.Generator().manual_seed(12)
    x = torch.randn(tokens, in_f, generator=g).to(torch.bfloat16).cuda().requires_grad_(True)
    dy = (1e-3 * torch.randn(tokens, out_f, generator=g)).to(torch.bfloat16).cuda()
    y = layer(x)
    y.backward(dy)
    torch.cuda.synchronize()
    b200.check_gemm_status(x.device)
    assert len(draws) == 2

    w = layer.weight.detach().float().cpu()
    xh, dyh = x.detach().float().cpu(), dy.float().cpu()
    ax, aw, ady = float(xh.abs().max()), float(w.abs().max()), float(dyh.abs().max())
    qx = oracle_quantize(xh, block=16, blocking=o.BLOCK_ROW, amax=ax)
    qw = oracle_quantize(w, block=16, blocking=o.BLOCK_2D, amax=aw)
    yo = o.gemm_issue_rz(qx["encoded"], qw["encoded"], snap=True, alpha_value=o.alpha(np.float32(ax), np.float32(aw), 448.0, 448.0))
    assert np.array_equal(to_np(y), bf16_round(yo))
    qdy = oracle_quantize(dyh, block=16, blocking=o.BLOCK_ROW, amax=ady, sr=True, bits=draws[0])
    dxo = o.gemm_issue_rz(qdy["encoded"], np.ascontiguousarray(qw["encoded"].T), snap=True,
                          alpha_value=o.alpha(np.float32(ady), np.float32(aw), 448.0, 448.0))
    assert np.array_equal(to_np(x.grad), bf16_round(dxo))
    # weight gradient: both operands transformed along the tokens, D=1 amax of the transformed tensors
    dyt = o.rht_b16(np.ascontiguousarray(dyh.numpy().T))
    xt = o.rht_b16(np.ascontiguousarray(xh.numpy().T))
    adyt, axt = float(np.abs(dyt).max()), float(np.abs(xt).max())
    qdyt = oracle_quantize(torch.from_numpy(dyt), block=16, blocking=o.BLOCK_ROW, amax=adyt, sr=True,
                           bits=draws[1].t().contiguous())
    qxt = oracle_quantize(torch.from_numpy(xt), block=16, blocking=o.BLOCK_ROW, amax=axt)
    dwo = o.gemm_issue_rz(qdyt["encoded"], qxt["encoded"], snap=True,
                          alpha_value=o.alpha(np.float32(adyt), np.float32(axt), 448.0, 448.0))
    assert np.array_equal(to_np(layer.weight.grad), dwo)
