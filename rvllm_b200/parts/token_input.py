"""An input that depends on the token's id alone, added to the stream at the end of a layer.

    e = table[token][column : column + dim]        one table for all layers, each layer its own columns
    g = gelu_tanh(W_gate x) * e                    x: the stream itself (no norm in front)
    y = W_proj g;   x <- x + y / sqrt(mean(y^2) + eps) * w

`token_table_rows` is the hook that looks the step's tokens up in the table ONCE per step (tensor named in full, as
the checkpoint names it) and leaves the rows in `ctx.extras[key]`; `token_side_input` is the per-layer part, a
feed-forward by interface, that reads its columns of those rows.  The norm's weight is a plain one.
"""
from __future__ import annotations

import torch

from .base import FEED_FORWARDS, HOOKS, Part, TensorSpec
from .linear import Linear


class TokenTableRows(Part):
    names_in_full = True

    def __init__(self, rows: int, width: int, tensor: str, key: str):
        self.rows, self.width, self.tensor, self.key = rows, width, tensor, key
        self.table = None

    def tensor_specs(self):
        return {self.tensor: TensorSpec((self.rows, self.width), "matrix")}

    def bind(self, get):
        self.table = get(self.tensor)

    def __call__(self, x, ctx):
        ctx.extras[self.key] = ctx.kernels.gather_rows(self.table, ctx.token_ids)
        return x


class TokenSideInput(Part):
    def __init__(self, hidden_size: int, dim: int, column: int, eps: float, table: str):
        self.hidden_size, self.dim, self.column, self.eps, self.table = hidden_size, dim, column, eps, table
        self.gate = Linear(hidden_size, [dim], ["gate"], suffix="")
        self.proj = Linear(dim, [hidden_size], ["proj"], suffix="")
        self.norm = None

    def tensor_specs(self):
        return {**self.gate.tensor_specs(), **self.proj.tensor_specs(), "norm": TensorSpec((self.hidden_size,), "norm")}

    def bind(self, get):
        self.gate.bind(get)
        self.proj.bind(get)
        self.norm = get("norm")

    def __call__(self, x, ctx, residual=None, out_dtype=None):
        """x: the stream in the activations' type; residual: the float32 stream, updated in place."""
        k = ctx.kernels
        g = self.gate(x, ctx, out_dtype=torch.float32)
        g = k.gelu_mul_columns(g, ctx.extras[self.table], self.column, x.dtype)
        y = self.proj(g, ctx, out_dtype=torch.float32)
        return k.residual_rmsnorm(y, self.norm, self.eps, residual, None)[0]


HOOKS.register("token_table_rows", TokenTableRows)
FEED_FORWARDS.register("token_side_input", TokenSideInput)
