"""Selective state-space mixer with one state row per channel ("mamba1").

    [u | z] = W_in h                                  u, z: inner channels each
    u <- silu(causal convolution per channel (taps, bias))
    [d | B | C] = W_x u                               d: dt_rank,  B, C: state
    dt = softplus(W_dt d + b_dt)                      one step size per channel
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n,   A = -exp(A_log)  [inner, state]
    y_c = sum_n S[c, n] C_n + D_c u_c;   out = W_o (y * silu(z))

A request keeps, in one row of a float32 state tensor, S ([inner][state]) and behind it the convolution's last
taps - 1 inputs; the cache manager zeroes the row when the slot is handed out.  B, C, the step sizes, the decays,
the state and the sums are float32; the products and the convolution's result have the activations' type.  A is
formed once, in float32, when the tensors are bound.  Nothing is read on the host, so a decode step can be captured.
"""
from __future__ import annotations

import torch

from .base import MIXERS, Part, StateNeed, TensorSpec
from .linear import Linear


class Mamba1Mixer(Part):
    def __init__(self, hidden_size: int, inner: int, state: int, dt_rank: int, conv: int):
        from ..errors import ConfigError
        problems = []
        if not 1 <= conv <= 16:
            problems.append(f"the convolution has 1 to 16 taps, got {conv}")
        if state > 256:
            problems.append(f"the state dimension is at most 256, got {state}")
        if problems:
            raise ConfigError(problems, "mamba1 mixer")
        self.hidden_size, self.inner, self.state, self.dt_rank, self.taps = hidden_size, inner, state, dt_rank, conv
        self.in_proj = Linear(hidden_size, [2 * inner], ["in"], suffix="")
        self.x_proj = Linear(inner, [dt_rank + 2 * state], ["x"], suffix="")
        self.dt_proj = Linear(dt_rank, [inner], ["dt"], suffix="")
        self.out = Linear(inner, [hidden_size], ["o"], suffix="")
        self.ssm_floats = inner * state
        self.conv_w = self.conv_b = self.dt_bias = self.a = self.d_skip = None

    def tensor_specs(self):
        return {**self.in_proj.tensor_specs(), **self.x_proj.tensor_specs(), **self.dt_proj.tensor_specs(),
                **self.out.tensor_specs(), "conv": TensorSpec((self.inner, self.taps), "conv_taps"),
                "conv.b": TensorSpec((self.inner,), "bias"), "dt.b": TensorSpec((self.inner,), "bias"),
                "A_log": TensorSpec((self.inner, self.state), "bias"), "D": TensorSpec((self.inner,), "norm")}

    def bind(self, get):
        for lin in (self.in_proj, self.x_proj, self.dt_proj, self.out):
            lin.bind(get)
        self.conv_w, self.conv_b = get("conv"), get("conv.b")
        # what enters the recurrence is float32
        self.dt_bias, self.d_skip = get("dt.b").float().contiguous(), get("D").float().contiguous()
        self.a = (-torch.exp(get("A_log").float())).contiguous()

    def cache_need(self):
        return StateNeed((self.ssm_floats + (self.taps - 1) * self.inner,), "float32")

    def __call__(self, x, ctx, cache, residual=None, write_cache=True, out_dtype=None):
        k = ctx.kernels
        proj = self.in_proj(x, ctx, out_dtype=torch.float32)                       # [u | z]
        u = k.causal_conv_silu(proj, 0, self.inner, self.conv_w, self.conv_b, ctx.token_seq, ctx.cu_seqlens,
                               ctx.state_slots, cache.state, self.ssm_floats, x.dtype)
        dbc = self.x_proj(u, ctx, out_dtype=torch.float32)                         # [d | B | C]
        d = k.column_slice(dbc, 0, self.dt_rank, x.dtype)
        dt_raw = self.dt_proj(d, ctx, out_dtype=torch.float32)
        y = k.selective_scan(u, dt_raw, self.dt_bias, self.a, dbc, self.dt_rank, self.dt_rank + self.state, self.d_skip,
                             proj, self.inner, ctx.cu_seqlens, ctx.state_slots, cache.state, x.dtype)
        return self.out(y, ctx, residual=residual, out_dtype=out_dtype)


MIXERS.register("mamba1", Mamba1Mixer)
