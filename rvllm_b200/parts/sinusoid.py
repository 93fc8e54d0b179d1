"""Sinusoidal position vectors added to the embedded tokens.

    x <- x * input_scale + pe(p),   pe(p)[2i] = sin(p w_i),  pe(p)[2i + 1] = cos(p w_i),  w_i = base^(-2i / width)

The frequencies are computed in float64 and handed to the kernel as such: it forms the angle p * w_i in double
precision, brings it into one turn, and takes sine and cosine of that in float32, so that the vector of a late
position is as exact as that of an early one.  The result is float32 (it starts a float32 residual stream).
"""
from __future__ import annotations

import torch

from .base import POSITION_ENCODINGS, Part


class SinusoidalEncoding(Part):
    def __init__(self, width: int, base: float = 10000.0, input_scale: float = 1.0):
        self.width, self.base, self.input_scale = width, float(base), float(input_scale)
        self.frequencies = torch.tensor([self.base ** (-2.0 * i / width) for i in range((width + 1) // 2)], dtype=torch.float64)

    def prepare(self, max_len: int, device) -> None:
        self.frequencies = self.frequencies.to(device)

    def rotation_tables(self):
        return None

    def on_embeddings(self, x, ctx):
        return ctx.kernels.scale_add_sinusoid(x, ctx.positions, self.frequencies, self.input_scale)


POSITION_ENCODINGS.register("sinusoidal", SinusoidalEncoding)
