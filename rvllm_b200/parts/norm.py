"""Norms of a layer.

RMSNorm: y = x / sqrt(mean(x^2) + eps) * gamma, arithmetic in float; gamma is the stored weight, or one plus
the stored weight for checkpoints that keep it around zero (`unit_offset`).

v3/crates/rvllm-fused/src/reference.rs:12-24 and kernels/fused_rmsnorm_fp8_quant.cu:61-84 of
the reference; eps comes from the configuration (the reference hard-codes 1e-6 in two tails,
v3/crates/rvllm-runtime/src/bring_up.rs:1219 - not followed).
"""
from __future__ import annotations

from .base import NORMS, Part, TensorSpec


class RMSNorm(Part):
    """`tensor` is the name of the weight below the part's prefix ("weight" in most checkpoints; "" where the
    prefix itself names the tensor).  `unit_offset`: the checkpoint stores gamma - 1; the sum is formed once, in
    float32, when the tensor is bound."""

    def __init__(self, size: int, eps: float, tensor: str = "weight", unit_offset: bool = False):
        self.size, self.eps, self.tensor, self.unit_offset = size, eps, tensor, unit_offset
        self.weight = None

    def tensor_specs(self):
        return {self.tensor: TensorSpec((self.size,), "norm")}

    def bind(self, get):
        self.weight = get(self.tensor)
        if self.unit_offset:
            self.weight = (self.weight.float() + 1.0).contiguous()

    def __call__(self, x, ctx):
        return ctx.kernels.rmsnorm(x, self.weight, self.eps)

    def as_rms(self):
        """(gamma, eps) for a part that applies this norm to its own input (see parts/block.py)."""
        return self.weight, self.eps


NORMS.register("rmsnorm", RMSNorm)


class DynamicTanh(Part):
    """y = tanh(alpha x) * weight + bias, element by element: a norm that forms no statistic of the row.  `alpha` is one
    number, stored beside the weight as `<tensor>.alpha`; the bias as `<tensor>.b`.  Arithmetic in float32; the three
    tensors are kept in float32 whatever the engine's type."""

    def __init__(self, size: int, tensor: str = "weight", bias_suffix: str = ".b", alpha_suffix: str = ".alpha"):
        self.size, self.tensor, self.bias_name, self.alpha_name = size, tensor, tensor + bias_suffix, tensor + alpha_suffix
        self.weight = self.bias = self.alpha = None

    def tensor_specs(self):
        return {self.tensor: TensorSpec((self.size,), "norm"), self.bias_name: TensorSpec((self.size,), "bias"),
                self.alpha_name: TensorSpec((), "unit_scale")}

    def bind(self, get):
        self.weight, self.bias = get(self.tensor).float().contiguous(), get(self.bias_name).float().contiguous()
        self.alpha = get(self.alpha_name).float().reshape(1).contiguous()

    def __call__(self, x, ctx):
        return ctx.kernels.dynamic_tanh(x, *self.as_dyt(), out_dtype=ctx.extras.get("activation_dtype", x.dtype))

    def as_dyt(self):
        """(alpha [1], weight, bias), float32, for a block that applies this norm inside a fused kernel."""
        return self.alpha, self.weight, self.bias


NORMS.register("dynamic_tanh", DynamicTanh)
