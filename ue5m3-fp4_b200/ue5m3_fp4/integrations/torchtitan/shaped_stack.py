"""A Nemotron-H-8B-SHAPED hybrid stack for throughput measurements of the FP4 linears under
data parallelism.

It has the reported model's 52-layer pattern (selection.py: Mamba2 / MLP / four self-attention
layers), hidden width 4096, the 112 internal linears with their real shapes and module names
(``layers.{i}.mixer.{in_proj,out_proj,up_proj,down_proj,q_proj,k_proj,v_proj,o_proj}``; shapes
from integrations/torchtitan/nemotron_h.py:166-182 of the reference), an embedding and an
``lm_head`` that the converter turns into the FP32 output head - so
``convert_reported_nemotron_h`` accepts it unchanged and every quantizer, GEMM and amax sample
of a training step runs at its real size.

What it is NOT: the mixers between the linears are cheap stand-ins, because the selective-scan
and causal-conv kernels of Mamba2 are separate libraries that are not part of this package.
The Mamba2 stand-in gates the two 8192-wide streams of ``in_proj`` (silu(z) * x) and adds the
B, C and dt columns onto the first 2176 channels, so that every output column of ``in_proj``
receives a gradient of the same order of magnitude; attention is torch's scaled-dot-product attention (causal, 32 query heads over 4
key/value heads of width 128, the reported k/v width 512); the MLP is up_proj ->
squared ReLU -> down_proj as in the model.  Outputs of this stack mean nothing; its cost profile
(FLOPs in the 112 linears, bytes of weights and gradients, number of amax samples) is the
model's.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn
from torch.nn import functional as F

from ue5m3_fp4.integrations.torchtitan.selection import (REPORTED_NEMOTRON_H_8B_PATTERN,
                                                          REPORTED_NEMOTRON_H_LAYER_COUNT)


@dataclass(frozen=True)
class ShapedConfig:
    """Widths of the reported 8B model; smaller values give a same-pattern toy for tests."""

    hidden_size: int = 4096
    intermediate_size: int = 21504          # MLP
    mamba_inner: int = 8192                 # z and x streams of in_proj; input width of out_proj
    mamba_extra: int = 2 * 1024 + 128       # B, C (8 groups x 128 states each) and dt (128 heads)
    attention_heads: int = 32
    kv_heads: int = 4
    head_dim: int = 128
    vocab_size: int = 131072
    num_hidden_layers: int = REPORTED_NEMOTRON_H_LAYER_COUNT
    hybrid_override_pattern: str = REPORTED_NEMOTRON_H_8B_PATTERN

    @property
    def in_proj_width(self) -> int:
        return 2 * self.mamba_inner + self.mamba_extra   # 18560 at the reported widths


class _RMSNorm(nn.Module):
    def __init__(self, width: int, device=None, dtype=None) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(width, device=device, dtype=dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.rms_norm(x, (x.shape[-1],), self.weight, 1e-5)


class _MambaStandIn(nn.Module):
    def __init__(self, c: ShapedConfig, device=None, dtype=None) -> None:
        super().__init__()
        self.inner, self.extra = c.mamba_inner, c.mamba_extra
        self.in_proj = nn.Linear(c.hidden_size, c.in_proj_width, bias=False, device=device, dtype=dtype)
        self.out_proj = nn.Linear(c.mamba_inner, c.hidden_size, bias=False, device=device, dtype=dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        z, u, rest = self.in_proj(x).split((self.inner, self.inner, self.extra), dim=-1)
        mixed = F.silu(z) * u
        mixed = torch.cat((mixed[..., :self.extra] + rest, mixed[..., self.extra:]), dim=-1)
        return self.out_proj(mixed)


class _Attention(nn.Module):
    def __init__(self, c: ShapedConfig, device=None, dtype=None) -> None:
        super().__init__()
        self.heads, self.kv_heads, self.head_dim = c.attention_heads, c.kv_heads, c.head_dim
        q_width, kv_width = c.attention_heads * c.head_dim, c.kv_heads * c.head_dim
        self.q_proj = nn.Linear(c.hidden_size, q_width, bias=False, device=device, dtype=dtype)
        self.k_proj = nn.Linear(c.hidden_size, kv_width, bias=False, device=device, dtype=dtype)
        self.v_proj = nn.Linear(c.hidden_size, kv_width, bias=False, device=device, dtype=dtype)
        self.o_proj = nn.Linear(q_width, c.hidden_size, bias=False, device=device, dtype=dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        batch, seq, _ = x.shape
        q = self.q_proj(x).view(batch, seq, self.heads, self.head_dim).transpose(1, 2)
        k = self.k_proj(x).view(batch, seq, self.kv_heads, self.head_dim).transpose(1, 2)
        v = self.v_proj(x).view(batch, seq, self.kv_heads, self.head_dim).transpose(1, 2)
        out = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        return self.o_proj(out.transpose(1, 2).reshape(batch, seq, self.heads * self.head_dim))


class _MLP(nn.Module):
    def __init__(self, c: ShapedConfig, device=None, dtype=None) -> None:
        super().__init__()
        self.up_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=False, device=device, dtype=dtype)
        self.down_proj = nn.Linear(c.intermediate_size, c.hidden_size, bias=False, device=device, dtype=dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(F.relu(self.up_proj(x)).square())


class _Layer(nn.Module):
    def __init__(self, kind: str, c: ShapedConfig, device=None, dtype=None) -> None:
        super().__init__()
        self.norm = _RMSNorm(c.hidden_size, device=device, dtype=dtype)
        self.mixer = {"M": _MambaStandIn, "*": _Attention, "-": _MLP}[kind](c, device=device, dtype=dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x + self.mixer(self.norm(x))


class NemotronHShapedStack(nn.Module):
    """Embedding -> 52 pre-norm residual layers -> norm -> lm_head; see the module docstring."""

    def __init__(self, config: ShapedConfig | None = None, *, device=None, dtype=torch.bfloat16) -> None:
        super().__init__()
        self.config = config or ShapedConfig()
        c = self.config
        if len(c.hybrid_override_pattern) != c.num_hidden_layers:
            raise ValueError("the layer pattern must name every layer")
        self.embed_tokens = nn.Embedding(c.vocab_size, c.hidden_size, device=device, dtype=dtype)
        self.layers = nn.ModuleList(_Layer(kind, c, device=device, dtype=dtype) for kind in c.hybrid_override_pattern)
        self.norm_f = _RMSNorm(c.hidden_size, device=device, dtype=dtype)
        self.lm_head = nn.Linear(c.hidden_size, c.vocab_size, bias=False, device=device, dtype=dtype)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        for module in self.modules():
            if isinstance(module, (nn.Linear, nn.Embedding)):
                module.weight.normal_(0.0, 0.02)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        x = self.embed_tokens(input_ids)
        for layer in self.layers:
            x = layer(x)
        return self.lm_head(self.norm_f(x))

    def fp4_linear_flops_per_token(self) -> int:
        """Forward + backward multiply-add FLOPs of the 112 internal linears per token (6 per weight)."""

        total = 0
        for name, module in self.named_modules():
            if ".mixer." in name and hasattr(module, "in_features") and hasattr(module, "out_features"):
                total += 6 * module.in_features * module.out_features
        return total


__all__ = ["NemotronHShapedStack", "ShapedConfig"]
