"""Hooks: small steps on the float32 logits or on the residual stream that belong to no layer.

`logit_softcap`   logits <- cap * tanh(logits / cap).
`stream_offset`   in front of a run entry: x <- x (+ the embedding output) + table[index], where `table` is a
                  tensor [rows, width] of the checkpoint named in full (several entries share it, each with its row).
                  This is what a model that runs a span of its layers several times adds at the start of each pass:
                  the embedded tokens again, and a vector that tells the passes apart.  The sum is float32.
`embedding_scale` on the embedded tokens: x <- scale * x, formed in float32 (the start of a float32 residual stream).
"""
from __future__ import annotations

import torch

from .base import HOOKS, Part, TensorSpec


class LogitSoftcap(Part):
    def __init__(self, cap: float):
        from ..errors import ConfigError
        if not cap > 0:
            raise ConfigError(f"the logit cap must be positive, got {cap}")
        self.cap = float(cap)

    def __call__(self, logits, ctx):
        return ctx.kernels.softcap(logits, self.cap)


class StreamOffset(Part):
    def __init__(self, width: int, rows: int, index: int, add_embedding: bool, tensor: str):
        from ..errors import ConfigError
        if not 0 <= index < rows:
            raise ConfigError(f"stream offset: row {index} of a table of {rows}")
        self.width, self.rows, self.index, self.add_embedding, self.tensor = width, rows, index, add_embedding, tensor
        self.needs_embedding_output = add_embedding
        self.table = None

    def tensor_specs(self):
        return {self.tensor: TensorSpec((self.rows, self.width), "bias")}

    def bind(self, get):
        self.table = get(self.tensor)

    def __call__(self, x, ctx):
        if x.dtype != torch.float32:
            x = x.float()
        emb = ctx.extras["embedding_output"] if self.add_embedding else None
        return ctx.kernels.stream_add(x, emb, self.table, self.index)


class EmbeddingScale(Part):
    def __init__(self, scale: float):
        self.scale = float(scale)

    def __call__(self, x, ctx):
        return ctx.kernels.scale_rows(x, self.scale)


HOOKS.register("embedding_scale", EmbeddingScale)
HOOKS.register("logit_softcap", LogitSoftcap)
HOOKS.register("stream_offset", StreamOffset)
