"""Grouped-query attention whose queries and keys are rotated and then made unit-RMS vectors, with a value size of its own,
a sliding window, a gate per head, and optionally another layer's keys and values.

    q = Wq h, k = Wk h  (per head `head_dim`),  v = Wv h  (per kv head `value_dim`);  no biases
    the leading rotary elements of every head of q and k are turned by the position (pairs (2i, 2i+1) or (i, i + half))
    q <- q / sqrt(mean(q^2) + eps),  k likewise                    per head, no weight, AFTER the rotation
    s = scale * (q . k);  a query at position i sees the keys j with 0 <= i - j < window (no window: j <= i);  softmax
    o_h <- o_h * sigmoid(Wg h)_h;  y = Wo [o_1 .. o_H]

What is cached is the key after rotation and norm, and the value.  A layer with `own_kv=False` has no key and value
matrices: it reads the cache slot of the layer that the run order names, with its own queries, window, scale and gate; that
slot keeps `kept_window` keys, the widest window among its readers (None: all keys; default: this layer's window).

A head's slot in the cache and in the attention kernels is `max(head_dim, value_dim)` wide; the shorter of key and value
is followed by zeros (which change no score and add nothing to a result), and the output matrix gets zero columns where a
head's slot is wider than its value.  One stacked product gives [q | k | v | gate logits] in float32; one kernel rotates,
normalises, writes the cache and applies the sigmoid.  Sizes and constants are parameters; tensors: q, k, v, g, o.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import MIXERS, KvCacheNeed, Part
from .linear import Linear


class UnitQkAttention(Part):
    PAIRS = ("neighbours", "halves")

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, scale: float,
                 eps: float, window: Optional[int] = None, kept_window="window", gate: bool = True,
                 pairs: str = "neighbours", own_kv: bool = True, position=None, suffix: str = ""):
        from ..errors import ConfigError
        problems = []
        if min(num_heads, num_kv_heads, head_dim, value_dim) < 1 or num_heads % max(num_kv_heads, 1):
            problems.append(f"{num_heads} query heads of {head_dim} on {num_kv_heads} key/value heads of {head_dim} / {value_dim}")
        if max(head_dim, value_dim) > 256:
            problems.append(f"key and value sizes are at most 256, got {head_dim} and {value_dim}")
        if pairs not in self.PAIRS:
            problems.append(f"rotation pairs {pairs!r} are not known ({', '.join(self.PAIRS)})")
        if kept_window == "window":                    # (None: the cache keeps every key, whatever this layer's window)
            kept_window = window
        if kept_window is not None and (window is None or kept_window < window):
            problems.append(f"the cache keeps {kept_window} keys but the window spans {window or 'all of them'}")
        if problems:
            raise ConfigError(problems, "unit-norm attention")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.value_dim, self.slot_dim = head_dim, value_dim, max(head_dim, value_dim)
        self.scale, self.eps, self.window, self.has_gate, self.pairs, self.own_kv = scale, eps, window, gate, pairs, own_kv
        self.kept_window = kept_window
        self.position = position
        outs, names = [num_heads * head_dim], ["q"]
        if own_kv:
            outs += [num_kv_heads * head_dim, num_kv_heads * value_dim]
            names += ["k", "v"]
        if gate:
            outs.append(num_heads)
            names.append("g")
        self.proj = Linear(hidden_size, outs, names, suffix=suffix)
        self.out = Linear(num_heads * value_dim, [hidden_size], ["o"], suffix=suffix)

    def tensor_specs(self):
        return {**self.proj.tensor_specs(), **self.out.tensor_specs()}

    def bind(self, get):
        self.proj.bind(get)
        self.out.bind(get)
        if self.slot_dim != self.value_dim:          # zero columns where a head's slot is wider than its value
            w = self.out.weight.view(self.hidden_size, self.num_heads, self.value_dim)
            wide = torch.zeros((self.hidden_size, self.num_heads, self.slot_dim), dtype=w.dtype, device=w.device)
            wide[:, :, :self.value_dim] = w
            self.out.weight = wide.view(self.hidden_size, self.num_heads * self.slot_dim).contiguous()

    def cache_need(self):
        return KvCacheNeed(self.num_kv_heads, self.slot_dim, self.kept_window)

    def __call__(self, x, ctx, cache, residual=None, write_cache=True, out_dtype=None):
        from ..errors import ConfigError
        if write_cache != self.own_kv:
            raise ConfigError("a unit-norm attention layer writes the cache exactly when it has key and value matrices of its own")
        k = ctx.kernels
        meta = ctx.attention[cache.group]
        tables = self.position.rotation_tables() if self.position is not None else None
        cos, sin = tables if tables is not None else (None, None)
        proj = self.proj(x, ctx, out_dtype=torch.float32)         # rounded once, after the rotation and the norm
        q, gate = k.qk_unit_prepare(proj, self.eps, ctx.positions, cos, sin, meta.slot_mapping, cache.kv, self.num_heads,
                                    self.num_kv_heads, self.head_dim, self.value_dim, self.slot_dim, x.dtype,
                                    halves=self.pairs == "halves", with_gate=self.has_gate, write_kv=write_cache)
        o = k.paged_attention(q, cache.kv, meta, self.num_heads, self.num_kv_heads, self.slot_dim, self.scale, self.window,
                              gate=gate)
        return self.out(o, ctx, residual=residual, out_dtype=out_dtype)


MIXERS.register("unit_qk_attention", UnitQkAttention)
