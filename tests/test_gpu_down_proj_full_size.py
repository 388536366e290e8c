"""The full FP4 linear of an MLP down-projection at its training size, block size 32:
X bf16 16384 x 21504 squared-ReLU, W bf16 4096 x 21504 ~ N(0, 0.02^2), dY bf16 16384 x 4096 ~
N(0, 1e-4^2); Y = X W^T, dX = dY W, dW = dY^T X with StochasticFast rounding on dY only, the 2048
target on dY for the dW GEMM (module layers.45.mixer.down_proj), and D = 50 delayed scaling over
120 optimizer steps with fresh seeded inputs every step.

All launches are full size.  The oracle checks sampled rows x columns of Y, dX and dW at a
refresh step (1), at a step that quantizes new data with the amax held since step 1 (50) and at
the third refresh (101); the cadence is checked over all 120 steps."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from gpu_helpers import bf16_round, oracle_quantize, to_np
from oracle import ue5m3_oracle as o

pytestmark = pytest.mark.gpu

TOKENS, IN_F, OUT_F, BLOCK = 16384, 21504, 4096, 32
NAME = "layers.45.mixer.down_proj"


def _inputs(step: int):
    g = torch.Generator(device="cuda").manual_seed(1000 + step)
    x = torch.relu(torch.randn(TOKENS, IN_F, device="cuda", generator=g)).square_().to(torch.bfloat16)
    dy = (1e-4 * torch.randn(TOKENS, OUT_F, device="cuda", generator=g)).to(torch.bfloat16)
    return x, dy


def test_down_proj_b32_full_size_over_120_steps(monkeypatch):
    import ue5m3_fp4.nn.linear as linear_module
    from ue5m3_fp4.backends import b200
    from ue5m3_fp4.nn import UE5M3Linear
    from ue5m3_fp4.recipe import UE5M3Recipe

    monkeypatch.setenv("UE5M3_GEMM_PATH", "fp4")
    recipe = UE5M3Recipe.proposed()
    recipe = UE5M3Recipe.from_dict({**recipe.to_dict(), "block_size": BLOCK, "name": "b32"})
    assert recipe.scale_target_for("wgrad_upstream_gradient", NAME) == 2048.0
    torch.manual_seed(0)
    layer = UE5M3Linear(IN_F, OUT_F, bias=False, recipe=recipe, backend="probe_matched", module_name=NAME,
                        device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        layer.weight.copy_(0.02 * torch.randn(OUT_F, IN_F, device="cuda"))
    draws = []
    original_draw = linear_module._draw_bits

    def recording_draw(reference):
        stream = original_draw(reference)
        draws.append(stream)
        return stream

    monkeypatch.setattr(linear_module, "_draw_bits", recording_draw)

    rows = torch.tensor([0, 1, 31, 32, 8191, 8192, 16352, 16383])            # tokens
    out_band, in_band = [0, 2048, 4064], [0, 10752, 21472]                   # first rows of 32 x 32 weight tiles
    out_cols = torch.cat([torch.arange(c, c + BLOCK) for c in out_band])      # 96 output features
    in_cols = torch.cat([torch.arange(c, c + BLOCK) for c in in_band])        # 96 input features
    w_host = layer.weight.detach().float().cpu()
    held = {}

    for step in range(1, 121):
        layer.scale_state.begin_step(step)
        x, dy = _inputs(step)
        x.requires_grad_(True)
        draws.clear()
        y = layer(x)
        y.backward(dy)
        if step in (1, 50, 101):
            torch.cuda.synchronize()
            b200.check_gemm_status(x.device)
            entries = {e["role"]: e for e in layer.scale_state.report()["entries"]}
            expect_refresh = 1 if step < 51 else 51 if step < 101 else 101
            assert all(e["last_refresh_step"] == expect_refresh for e in entries.values())
            ax, aw, ady = (entries[k]["reference_amax"] for k in ("activation", "weight", "upstream_gradient"))
            if step in (1, 101):  # a refresh step samples the current tensors
                assert ax == float(x.detach().float().abs().max()) and ady == float(dy.float().abs().max())
                held[step] = (ax, ady)
            else:                 # step 50 still quantizes with what step 1 sampled
                assert (ax, ady) == held[1]
            assert len(draws) == 2
            bits_dgrad = draws[0].materialize(dy.shape)
            bits_wgrad = draws[1].materialize(dy.shape)
            xd = x.detach()

            # Y[rows, out_cols]: X rows (1 x 32 blocks) . W bands (32 x 32 tiles)
            qx = oracle_quantize(xd[rows.cuda()].float().cpu(), block=BLOCK, blocking=o.BLOCK_ROW, amax=ax)
            enc_w = np.concatenate([oracle_quantize(w_host[c:c + BLOCK], block=BLOCK, blocking=o.BLOCK_2D, amax=aw)["encoded"]
                                    for c in out_band])
            alpha = o.alpha(np.float32(ax), np.float32(aw), 448.0, 448.0)
            expect = bf16_round(o.gemm_issue_rz(qx["encoded"], enc_w, snap=True, alpha_value=alpha))
            assert np.array_equal(to_np(y.detach()[rows.cuda()][:, out_cols.cuda()]), expect), ("Y", step)

            # dX[rows, in_cols]: dY rows (stochastic, first draw) . W^T (the same 32 x 32 tiles, read along out)
            qdy = oracle_quantize(dy[rows.cuda()].float().cpu(), block=BLOCK, blocking=o.BLOCK_ROW, amax=ady, sr=True,
                                  bits=bits_dgrad[rows.cuda()].cpu())
            enc_wt = np.concatenate([
                np.ascontiguousarray(oracle_quantize(w_host[:, c:c + BLOCK], block=BLOCK, blocking=o.BLOCK_2D, amax=aw)["encoded"].T)
                for c in in_band])
            alpha = o.alpha(np.float32(ady), np.float32(aw), 448.0, 448.0)
            expect = bf16_round(o.gemm_issue_rz(qdy["encoded"], enc_wt, snap=True, alpha_value=alpha))
            assert np.array_equal(to_np(x.grad[rows.cuda()][:, in_cols.cuda()]), expect), ("dX", step)

            # dW[out_cols, in_cols]: dY^T (stochastic, second draw, T = 2048) . X^T, both blocked along the tokens
            qdyt = oracle_quantize(dy[:, out_cols.cuda()].float().cpu(), block=BLOCK, blocking=o.BLOCK_COL, amax=ady,
                                   target=2048.0, sr=True, bits=bits_wgrad[:, out_cols.cuda()].cpu())
            qxt = oracle_quantize(xd[:, in_cols.cuda()].float().cpu(), block=BLOCK, blocking=o.BLOCK_COL, amax=ax)
            alpha = o.alpha(np.float32(ady), np.float32(ax), 2048.0, 448.0)
            expect = bf16_round(o.gemm_issue_rz(np.ascontiguousarray(qdyt["encoded"].T), np.ascontiguousarray(qxt["encoded"].T),
                                                snap=True, alpha_value=alpha))
            got = to_np(layer.weight.grad[out_cols.cuda()][:, in_cols.cuda()])
            assert np.array_equal(got, expect), ("dW", step)
            del bits_dgrad, bits_wgrad
        layer.weight.grad = None
        del x, dy, y

    torch.cuda.synchronize()
    b200.check_gemm_status(torch.device("cuda", 0))
    for entry in layer.scale_state.report()["entries"]:
        assert (entry["refreshes"], entry["reuses"], entry["last_refresh_step"]) == (3, 117, 101)
