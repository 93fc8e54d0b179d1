"""Gated feed-forward: down( act(gate(x)) * up(x) ), act = SiLU or the tanh form of GELU, the
residual added in the last product's epilogue.  gate and up are one stacked product whose rows are [gate | up]
(kernels/fused_silu_fp8_quant.cu:52-56 and v3/crates/rvllm-runtime/src/layer_exec.rs:476-522
of the reference)."""
from __future__ import annotations

import torch

from .base import FEED_FORWARDS, Part
from .linear import Linear


class GatedMLP(Part):
    takes_input_norm = True           # the gate/up product can apply the layer's RMSNorm itself

    ACTIVATIONS = ("silu", "gelu_tanh")

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 names=("gate_proj", "up_proj", "down_proj"), suffix: str = ".weight"):
        from ..errors import ConfigError
        if activation not in self.ACTIVATIONS:
            raise ConfigError(f"gated MLP activation {activation!r} is not supported (known: {', '.join(self.ACTIVATIONS)})")
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        self.gate_up = Linear(hidden_size, [intermediate_size, intermediate_size], list(names[:2]), suffix=suffix)
        self.down = Linear(intermediate_size, [hidden_size], [names[2]], suffix=suffix)

    def tensor_specs(self):
        return {**self.gate_up.tensor_specs(), **self.down.tensor_specs()}

    def bind(self, get):
        self.gate_up.bind(get)
        self.down.bind(get)

    def __call__(self, x, ctx, residual=None, input_norm=None, out_dtype=None):
        if self.activation == "silu":
            h = ctx.kernels.gate_up_silu(x, self.gate_up.weight, norm=input_norm)
        else:
            h = ctx.kernels.gate_up_act(x, self.gate_up.weight, self.activation, norm=input_norm)
        return self.down(h, ctx, residual=residual, out_dtype=out_dtype)


FEED_FORWARDS.register("gated_mlp", GatedMLP)


class ClampedGluMLP(Part):
    """down( g sigmoid(alpha g) (u + 1) ) with g = min(gate(x), limit) and u = clamp(up(x), -limit, limit); every
    product has a bias.  gate and up are one stacked product [gate | up] that leaves its kernel in float32; the
    activation kernel rounds once."""

    def __init__(self, hidden_size: int, intermediate_size: int, limit: float, alpha: float = 1.702,
                 names=("gate", "up", "down"), suffix: str = "", bias_suffix: str = ".b"):
        from ..errors import ConfigError
        if not limit > 0:
            raise ConfigError(f"the clamp of the gated feed-forward must be positive, got {limit}")
        self.hidden_size, self.intermediate_size, self.limit, self.alpha = hidden_size, intermediate_size, float(limit), float(alpha)
        self.gate_up = Linear(hidden_size, [intermediate_size, intermediate_size], list(names[:2]), bias=True, suffix=suffix,
                              bias_suffix=bias_suffix)
        self.down = Linear(intermediate_size, [hidden_size], [names[2]], bias=True, suffix=suffix, bias_suffix=bias_suffix)

    def tensor_specs(self):
        return {**self.gate_up.tensor_specs(), **self.down.tensor_specs()}

    def bind(self, get):
        self.gate_up.bind(get)
        self.down.bind(get)

    def __call__(self, x, ctx, residual=None, out_dtype=None):
        gu = self.gate_up(x, ctx, out_dtype=torch.float32)
        h = ctx.kernels.act_mul(gu, "swiglu_clamp", x.dtype, limit=self.limit, alpha=self.alpha)
        return self.down(h, ctx, residual=residual, out_dtype=out_dtype)


FEED_FORWARDS.register("clamped_glu_mlp", ClampedGluMLP)
