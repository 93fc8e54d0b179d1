"""Gated delta rule: a linear-attention mixer whose state is corrected towards each new value.

    q = Wq h, k = Wk h  (qk_heads x head_dim),  v = Wv h  (heads x value_dim);  value head i uses q/k head i // (heads / qk_heads)
    q, k, v <- silu(causal convolution per channel (taps, no bias))
    q <- q / sqrt(sum(q^2) + 1e-6) * head_dim^(-1/2),   k <- k / sqrt(sum(k^2) + 1e-6)         per head
    beta = sigmoid(Wb h),   g = exp(-exp(A_log) softplus(Wa h + dt_bias))                       one each per head
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q                             S: head_dim x value_dim
    o <- o / sqrt(mean(o^2) + eps) * w * silu(Wg h);   y = Wo o                                 w: value_dim, shared by the heads

One stacked product gives [q | k | v | gate | beta logits | decay logits] in float32.  A request keeps, in one row of
a float32 state tensor, S ([heads][head_dim][value_dim]) and behind it the convolutions' last taps - 1 inputs (the three
convolutions are one over the channels q | k | v).  The unit norms, beta, the decay, the state and its sums and the
output norm are float32; the products and the convolutions' results have the activations' type.
"""
from __future__ import annotations

import torch

from .base import MIXERS, Part, StateNeed, TensorSpec
from .linear import Linear


class GatedDeltaRule(Part):
    def __init__(self, hidden_size: int, heads: int, qk_heads: int, head_dim: int, value_dim: int, conv: int, eps: float,
                 unit_eps: float = 1e-6):
        from ..errors import ConfigError
        problems = []
        if heads % qk_heads:
            problems.append(f"{heads} value heads cannot share {qk_heads} query/key heads")
        if not 1 <= conv <= 16:
            problems.append(f"the convolution has 1 to 16 taps, got {conv}")
        if head_dim > 256 or value_dim > 1024:
            problems.append(f"head_dim is at most 256 and value_dim at most 1024, got {head_dim} and {value_dim}")
        if problems:
            raise ConfigError(problems, "gated delta rule")
        self.hidden_size, self.heads, self.qk_heads, self.head_dim, self.value_dim = hidden_size, heads, qk_heads, head_dim, value_dim
        self.taps, self.eps, self.unit_eps = conv, eps, unit_eps
        self.qk_dim, self.v_dim = qk_heads * head_dim, heads * value_dim
        self.channels = 2 * self.qk_dim + self.v_dim                       # what passes the convolution: q | k | v
        self.proj = Linear(hidden_size, [self.qk_dim, self.qk_dim, self.v_dim, self.v_dim, heads, heads],
                           ["q", "k", "v", "g", "b", "a"], suffix="")
        self.out = Linear(self.v_dim, [hidden_size], ["o"], suffix="")
        self.state_floats = heads * head_dim * value_dim
        self.conv_w = self.a_log = self.dt_bias = self.norm = None

    def tensor_specs(self):
        return {**self.proj.tensor_specs(), **self.out.tensor_specs(),
                "q.conv": TensorSpec((self.qk_dim, self.taps), "conv_taps"), "k.conv": TensorSpec((self.qk_dim, self.taps), "conv_taps"),
                "v.conv": TensorSpec((self.v_dim, self.taps), "conv_taps"), "A_log": TensorSpec((self.heads,), "bias"),
                "dt_bias": TensorSpec((self.heads,), "bias"), "norm": TensorSpec((self.value_dim,), "norm")}

    def bind(self, get):
        self.proj.bind(get)
        self.out.bind(get)
        self.conv_w = torch.cat([get("q.conv"), get("k.conv"), get("v.conv")], dim=0).contiguous()
        self.a_log, self.dt_bias = get("A_log").float().contiguous(), get("dt_bias").float().contiguous()
        self.norm = get("norm")

    def cache_need(self):
        return StateNeed((self.state_floats + (self.taps - 1) * self.channels,), "float32")

    def __call__(self, x, ctx, cache, residual=None, write_cache=True, out_dtype=None):
        k = ctx.kernels
        proj = self.proj(x, ctx, out_dtype=torch.float32)
        qkv = k.causal_conv_silu(proj, 0, self.channels, self.conv_w, None, ctx.token_seq, ctx.cu_seqlens, ctx.state_slots,
                                 cache.state, self.state_floats, x.dtype)
        gate_col = self.channels
        o = k.delta_rule(qkv, proj, gate_col + self.v_dim, gate_col + self.v_dim + self.heads, self.a_log, self.dt_bias,
                         ctx.cu_seqlens, ctx.state_slots, cache.state, self.heads, self.qk_heads, self.head_dim, self.value_dim,
                         self.unit_eps)
        o = k.head_norm_gate(o, self.norm, self.eps, proj, gate_col, self.heads, self.value_dim, x.dtype)
        return self.out(o, ctx, residual=residual, out_dtype=out_dtype)


MIXERS.register("gated_delta_rule", GatedDeltaRule)
