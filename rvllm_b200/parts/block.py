"""Arrangements of a layer's parts.

`prenorm_residual`: x + mixer(norm(x)), then + feed_forward(norm(.)); the additions happen in
the epilogue of each part's last product (v3/crates/rvllm-runtime/src/layer_exec.rs:189-205,
431-444, 460-474, 511-522 of the reference).

A mixer or feed-forward whose class sets `takes_input_norm = True` accepts `input_norm=(gamma,
eps)` and applies that RMSNorm to its input itself (its first product does it in its kernel for
few rows); the block then hands it the unnormalised x.  A norm offers this through `as_rms()`;
parts and norms without these attributes are combined the plain way."""
from __future__ import annotations

import torch

from .base import BLOCKS


class PreNormResidualBlock:
    ROLES = ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm")

    def __init__(self, parts):
        from ..errors import ConfigError
        if sorted(parts) != sorted(self.ROLES):
            raise ConfigError(f"the pre-norm residual block arranges the parts {', '.join(self.ROLES)}; got {', '.join(sorted(parts))}")
        self.mixer, self.feed_forward = parts["mixer"], parts["feed_forward"]
        self.mixer_norm, self.feed_forward_norm = parts["mixer_norm"], parts["feed_forward_norm"]

    @staticmethod
    def _handed_over(part, norm):
        if getattr(part, "takes_input_norm", False) and hasattr(norm, "as_rms"):
            return norm.as_rms()
        return None

    def __call__(self, x, ctx, cache, write_cache=True):
        norm = self._handed_over(self.mixer, self.mixer_norm)
        if norm is not None:
            x = self.mixer(x, ctx, cache, residual=x, write_cache=write_cache, input_norm=norm)
        else:
            x = self.mixer(self.mixer_norm(x, ctx), ctx, cache, residual=x, write_cache=write_cache)
        norm = self._handed_over(self.feed_forward, self.feed_forward_norm)
        if norm is not None:
            return self.feed_forward(x, ctx, residual=x, input_norm=norm)
        return self.feed_forward(self.feed_forward_norm(x, ctx), ctx, residual=x)


BLOCKS.register("prenorm_residual", PreNormResidualBlock)


class OutputNormResidualBlock:
    """`output_norm_residual`: x + norm(mixer(x)), then + norm(feed_forward(x)); the sublayers read the stream
    itself and the norm acts on what they return.  A layer may have no feed-forward.

    The stream x is float32 whatever the engine's type (`ModelSpec.residual_dtype`): the norm, the sum and
    the stream stay in 32 bits, and the kernel that adds also leaves the copy of the new stream in the
    activations' type that the next sublayer's products read.  The copy travels beside the stream in
    `ctx.extras`; a block that finds none (the first layer) makes one.  Sublayers are asked for a float32
    result (`out_dtype`), so that what is normalised was rounded nowhere after its last product."""
    ROLES = ("mixer", "mixer_norm")
    OPTIONAL = ("feed_forward", "feed_forward_norm")
    KEY = "rounded_stream"

    def __init__(self, parts):
        from ..errors import ConfigError
        names = set(parts)
        if not set(self.ROLES) <= names or not names <= set(self.ROLES + self.OPTIONAL) or \
                (("feed_forward" in names) != ("feed_forward_norm" in names)):
            raise ConfigError(f"the output-norm residual block arranges {', '.join(self.ROLES)} and, together, "
                              f"{', '.join(self.OPTIONAL)}; got {', '.join(sorted(parts))}")
        self.mixer, self.mixer_norm = parts["mixer"], parts["mixer_norm"]
        self.feed_forward, self.feed_forward_norm = parts.get("feed_forward"), parts.get("feed_forward_norm")
        for n in (self.mixer_norm, self.feed_forward_norm):
            if n is not None and not hasattr(n, "as_rms"):
                raise ConfigError("the output-norm residual block needs norms that offer `as_rms()` (an RMSNorm)")

    def _rounded(self, x, ctx, dtype):
        if dtype == torch.float32:
            return x
        kept = ctx.extras.get(self.KEY)
        if kept is not None and kept[0] is x:
            return kept[1]
        return x.to(dtype)

    def _add(self, x, y, norm, ctx, dtype):
        gamma, eps = norm.as_rms()
        x, h = ctx.kernels.residual_rmsnorm(y, gamma, eps, x, dtype)
        ctx.extras[self.KEY] = (x, h)
        return x

    def __call__(self, x, ctx, cache, write_cache=True):
        dtype = ctx.extras.get("activation_dtype", x.dtype)
        if x.dtype != torch.float32:
            x = x.float()
        h = self._rounded(x, ctx, dtype)
        x = self._add(x, self.mixer(h, ctx, cache, residual=None, write_cache=write_cache, out_dtype=torch.float32),
                      self.mixer_norm, ctx, dtype)
        if self.feed_forward is not None:
            h = self._rounded(x, ctx, dtype)
            x = self._add(x, self.feed_forward(h, ctx, residual=None, out_dtype=torch.float32), self.feed_forward_norm, ctx, dtype)
        return x


BLOCKS.register("output_norm_residual", OutputNormResidualBlock)


class SandwichNormResidualBlock:
    """`sandwich_norm_residual`: x + norm_out(mixer(norm_in(x))), then x + norm_out'(feed_forward(norm_in'(x))): every
    sublayer has a norm in front of it and one on what it returns.  A layer may have no feed-forward.  The norms of a layer
    are all RMSNorms (`as_rms()`) or all Dynamic-Tanh norms (`as_dyt()`).

    The stream x is float32 whatever the engine's type (`ModelSpec.residual_dtype`); sublayers are asked for a float32
    result, which is normalised and added in 32 bits.  One kernel does the sum and the norm in front of the NEXT sublayer
    of the layer (for RMSNorms two row statistics in one pass over the row), and leaves that sublayer's input in the
    activations' type."""
    ROLES = ("mixer", "mixer_norm", "mixer_out_norm")
    OPTIONAL = ("feed_forward", "feed_forward_norm", "feed_forward_out_norm")

    def __init__(self, parts):
        from ..errors import ConfigError
        names = set(parts)
        n_opt = sum(1 for r in self.OPTIONAL if r in names)
        if not set(self.ROLES) <= names or not names <= set(self.ROLES + self.OPTIONAL) or n_opt not in (0, len(self.OPTIONAL)):
            raise ConfigError(f"the sandwich-norm residual block arranges {', '.join(self.ROLES)} and, together, "
                              f"{', '.join(self.OPTIONAL)}; got {', '.join(sorted(parts))}")
        self.mixer, self.mixer_norm, self.mixer_out_norm = (parts[r] for r in self.ROLES)
        self.feed_forward, self.feed_forward_norm, self.feed_forward_out_norm = (parts.get(r) for r in self.OPTIONAL)
        norms = [n for n in (self.mixer_norm, self.mixer_out_norm, self.feed_forward_norm, self.feed_forward_out_norm) if n is not None]
        if all(hasattr(n, "as_rms") for n in norms):
            self.kind = "rms"
        elif all(hasattr(n, "as_dyt") for n in norms):
            self.kind = "dyt"
        else:
            raise ConfigError("the sandwich-norm residual block needs norms that all offer `as_rms()` (RMSNorm) or all "
                              "`as_dyt()` (Dynamic Tanh)")

    def _norm(self, k, norm, x, dtype):
        if self.kind == "rms":
            return k.rmsnorm(x, *norm.as_rms(), out_dtype=dtype)
        return k.dynamic_tanh(x, *norm.as_dyt(), out_dtype=dtype)

    def _add(self, k, norm, y, x, dtype, next_norm):
        """x + norm(y) and, with `next_norm`, that norm of the sum in `dtype`."""
        if self.kind == "rms":
            if next_norm is None:
                return k.residual_rmsnorm(y, *norm.as_rms(), x, None)[0], None
            return k.residual_rmsnorm(y, *norm.as_rms(), x, dtype, next_norm=next_norm.as_rms())
        return k.residual_dynamic_tanh(y, norm.as_dyt(), x, None if next_norm is None else next_norm.as_dyt(), dtype)

    def __call__(self, x, ctx, cache, write_cache=True):
        k = ctx.kernels
        dtype = ctx.extras.get("activation_dtype", x.dtype)
        if x.dtype != torch.float32:
            x = x.float()
        h = self._norm(k, self.mixer_norm, x, dtype)
        y = self.mixer(h, ctx, cache, residual=None, write_cache=write_cache, out_dtype=torch.float32)
        if self.feed_forward is None:
            return self._add(k, self.mixer_out_norm, y, x, dtype, None)[0]
        x, h = self._add(k, self.mixer_out_norm, y, x, dtype, self.feed_forward_norm)
        y = self.feed_forward(h, ctx, residual=None, out_dtype=torch.float32)
        return self._add(k, self.feed_forward_out_norm, y, x, dtype, None)[0]


BLOCKS.register("sandwich_norm_residual", SandwichNormResidualBlock)


class PreNormStreamResidualBlock:
    """`prenorm_stream_residual`: x + mixer(norm(x)), then x + feed_forward(norm(x)), on a float32 stream
    (`ModelSpec.residual_dtype`): the sublayers return float32, the sums are formed in 32 bits, and the kernel that
    adds a sublayer's result also writes what the next sublayer reads (the new stream under that sublayer's norm, in
    the activations' type).  A layer may have no feed-forward.  An optional last part `token_input` (a feed-forward
    by interface: `__call__(x, ctx, residual) -> residual + f(x)`) reads the stream ITSELF, not a normalised copy."""
    ROLES = ("mixer", "mixer_norm")
    OPTIONAL = ("feed_forward", "feed_forward_norm", "token_input")

    def __init__(self, parts):
        from ..errors import ConfigError
        names = set(parts)
        if not set(self.ROLES) <= names or not names <= set(self.ROLES + self.OPTIONAL) or \
                (("feed_forward" in names) != ("feed_forward_norm" in names)):
            raise ConfigError(f"the pre-norm stream block arranges {', '.join(self.ROLES)} and optionally "
                              f"{', '.join(self.OPTIONAL)}; got {', '.join(sorted(parts))}")
        self.mixer, self.mixer_norm = parts["mixer"], parts["mixer_norm"]
        self.feed_forward, self.feed_forward_norm = parts.get("feed_forward"), parts.get("feed_forward_norm")
        self.token_input = parts.get("token_input")
        for n in (self.mixer_norm, self.feed_forward_norm):
            if n is not None and not hasattr(n, "as_rms"):
                raise ConfigError("the pre-norm stream block needs norms that offer `as_rms()` (an RMSNorm)")

    def __call__(self, x, ctx, cache, write_cache=True):
        k = ctx.kernels
        dtype = ctx.extras.get("activation_dtype", x.dtype)
        if x.dtype != torch.float32:
            x = x.float()
        h = k.rmsnorm(x, *self.mixer_norm.as_rms(), out_dtype=dtype)
        y = self.mixer(h, ctx, cache, residual=None, write_cache=write_cache, out_dtype=torch.float32)
        if self.feed_forward is not None:
            x, h = k.stream_add_norm(x, y, self.feed_forward_norm.as_rms(), dtype)
            y = self.feed_forward(h, ctx, residual=None, out_dtype=torch.float32)
        if self.token_input is None:
            return k.stream_add_norm(x, y, None, None)[0]
        x, h = k.stream_add_norm(x, y, None, dtype)
        return self.token_input(h, ctx, residual=x)


BLOCKS.register("prenorm_stream_residual", PreNormStreamResidualBlock)
