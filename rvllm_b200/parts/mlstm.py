"""mLSTM: a matrix memory per head with exponential input and forget gates held stable by a running maximum.

    q = Wq h * head_dim^(-1/2),  k = Wk h  (heads x head_dim),  v = Wv h  (heads x value_dim)
    i = cap tanh((Wi h + bi) / cap),   f = logsigmoid(cap tanh((Wf h + bf) / cap))              one each per head, logarithms
    m_t = max(f + m_(t-1), i);   a = exp(f + m_(t-1) - m_t),  b = exp(i - m_t)                 m starts at 0
    S_t = a S_(t-1) + b k v^T;   n_t = a n_(t-1) + b k                                          S: head_dim x value_dim, both start at 0
    o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)
    o <- o / sqrt(mean(o^2) + eps) per head;   y = Wo (o * w * sigmoid(Wg h))                   w: heads x value_dim

One stacked product gives [q | k | v | gate | i | f] in float32.  A request keeps, in one row of a float32 state tensor,
[heads][head_dim][value_dim + 1] (the last column of a head is n: the memory of the constant value 1) and behind it m per
head; the cache manager zeroes the row when the slot is handed out, which is the state the recurrence starts from.  The
gates, their exponentials, the state, the normaliser and the output norm are float32.  Nothing is read on the host.
"""
from __future__ import annotations

import torch

from .base import MIXERS, Part, StateNeed, TensorSpec
from .linear import Linear


class MLstmMixer(Part):
    def __init__(self, hidden_size: int, heads: int, head_dim: int, value_dim: int, gate_cap: float, eps: float,
                 denominator_eps: float = 1e-6):
        from ..errors import ConfigError
        problems = []
        if min(heads, head_dim, value_dim) < 1:
            problems.append("sizes must be positive")
        if head_dim > 1024 or value_dim > 4096:
            problems.append(f"head_dim is at most 1024 and value_dim at most 4096, got {head_dim} and {value_dim}")
        if not gate_cap > 0:
            problems.append(f"the cap of the gates must be positive, got {gate_cap}")
        if problems:
            raise ConfigError(problems, "mlstm mixer")
        self.hidden_size, self.heads, self.head_dim, self.value_dim = hidden_size, heads, head_dim, value_dim
        self.gate_cap, self.eps, self.denominator_eps = float(gate_cap), eps, denominator_eps
        self.qk_dim, self.v_dim = heads * head_dim, heads * value_dim
        self.proj = Linear(hidden_size, [self.qk_dim, self.qk_dim, self.v_dim, self.v_dim, heads, heads],
                           ["q", "k", "v", "g", "i", "f"], suffix="")
        self.out = Linear(self.v_dim, [hidden_size], ["o"], suffix="")
        self.memory_floats = heads * head_dim * (value_dim + 1)
        self.i_bias = self.f_bias = self.norm = None

    def tensor_specs(self):
        return {**self.proj.tensor_specs(), **self.out.tensor_specs(), "i.b": TensorSpec((self.heads,), "bias"),
                "f.b": TensorSpec((self.heads,), "bias"), "norm": TensorSpec((self.v_dim,), "norm")}

    def bind(self, get):
        self.proj.bind(get)
        self.out.bind(get)
        self.i_bias, self.f_bias = get("i.b").float().contiguous(), get("f.b").float().contiguous()   # gates are float32
        self.norm = get("norm").float().contiguous()

    def cache_need(self):
        return StateNeed((self.memory_floats + self.heads,), "float32")

    def __call__(self, x, ctx, cache, residual=None, write_cache=True, out_dtype=None):
        k = ctx.kernels
        proj = self.proj(x, ctx, out_dtype=torch.float32)
        gate_col = 2 * self.qk_dim + self.v_dim
        raw, top = k.mlstm_scan(proj, gate_col + self.v_dim, gate_col + self.v_dim + self.heads, self.i_bias, self.f_bias,
                                ctx.cu_seqlens, ctx.state_slots, cache.state, self.heads, self.head_dim, self.value_dim,
                                self.gate_cap)
        y = k.mlstm_output(raw, top, self.norm, self.eps, self.denominator_eps, proj, gate_col, self.heads, self.head_dim,
                           self.value_dim, x.dtype, ctx.token_seq, ctx.cu_seqlens, ctx.state_slots, cache.state)
        return self.out(y, ctx, residual=residual, out_dtype=out_dtype)


MIXERS.register("mlstm", MLstmMixer)
