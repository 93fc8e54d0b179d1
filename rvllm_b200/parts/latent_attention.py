"""Latent attention: keys and values of all heads are projections of ONE low-rank row per token, and only
that row is cached.

    q = Wq h                            per head [dim unrotated | rot_dim rotated]
    [c' | r] = Wdkv h                   c = rms(c') * w  (kv_rank values), r: rot_dim values, one rotated key part for all heads
    k_h = [Wuk_h c | rot(r)],  v_h = Wuv_h c
    s = scale * (q_h . k_h), causal, softmax;  o_h = sigmoid(Wg h)_h * sum_j p_j v_hj;  y = Wo [o_1 .. o_H]

The rotation turns the pairs (2i, 2i + 1) - or, with `pairs="halves"`, (i, i + rotary_dim / 2) - of the leading
`rotary_dim` elements of the rotated part by position * base^(-2i / rotary_dim); the rest passes.  With `sink=True` the
softmax's denominator also holds exp(sink_h), a number per head that has neither key nor value (tensor `sink`).

What is computed is the same thing with the two up-projections moved out of the sum over the keys:

    q_h . (Wuk_h c_j) = (Wuk_h^T q_h) . c_j          sum_j p_j Wuv_h c_j = Wuv_h (sum_j p_j c_j)

so the cache holds one row [c | rot(r)] of kv_rank + rot_dim elements per token (one plane, one "kv head"), every
head's query becomes [Wuk_h^T q_h | rot(q_h rotated part)] of that width, the attention kernel reads the row's
leading kv_rank elements as the value, and Wuv_h is applied once per query to the kv_rank-wide result.  A step costs
the same whatever part of the context it attends to, and nothing per head is ever stored.

One stacked product gives [q | c' r | gate logits] in float32; one kernel normalises c', rotates, writes the cache row,
splits q and applies the sigmoid; two products per head (batched over the heads) absorb Wuk into the query and apply
Wuv to the result.  Sizes and constants are parameters; tensor names default to q, dkv, dkv.norm, uk, uv, g, o.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import MIXERS, KvCacheNeed, Part, TensorSpec
from .linear import Linear


class LatentAttention(Part):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, value_dim: int, kv_rank: int,
                 scale: float, eps: float, gate: bool = True, position=None, suffix: str = "", sink: bool = False,
                 pairs: str = "neighbours"):
        from ..errors import ConfigError
        problems = []
        if min(num_heads, head_dim, value_dim, kv_rank) < 1 or rot_dim < 0:
            problems.append("sizes must be positive")
        if rot_dim % 2:
            problems.append(f"the rotated part must have an even size, got {rot_dim}")
        if pairs not in ("neighbours", "halves"):
            problems.append(f"rotation pairs {pairs!r} are not known (neighbours, halves)")
        if kv_rank + rot_dim > 1024:
            problems.append(f"a cached row (kv_rank + rot_dim) holds at most 1,024 elements, got {kv_rank + rot_dim}")
        if problems:
            raise ConfigError(problems, "latent attention")
        self.hidden_size, self.num_heads, self.head_dim, self.rot_dim = hidden_size, num_heads, head_dim, rot_dim
        self.value_dim, self.kv_rank, self.scale, self.eps, self.has_gate = value_dim, kv_rank, scale, eps, gate
        self.position, self.has_sink, self.pairs = position, sink, pairs
        self.q_head = head_dim + rot_dim                 # a head's slice of the query product
        self.row = kv_rank + rot_dim                     # a cached row, and a head's absorbed query
        outs, names = [num_heads * self.q_head, self.row], ["q", "dkv"]
        if gate:
            outs.append(num_heads)
            names.append("g")
        self.qdg = Linear(hidden_size, outs, names, suffix=suffix)
        self.out = Linear(num_heads * value_dim, [hidden_size], ["o"], suffix=suffix)
        self.c_norm = self.uk_t = self.uv = self.sink = None

    def tensor_specs(self):
        sink = {"sink": TensorSpec((self.num_heads,), "bias")} if self.has_sink else {}
        return {**self.qdg.tensor_specs(), **self.out.tensor_specs(), **sink,
                "dkv.norm": TensorSpec((self.kv_rank,), "norm"),
                "uk": TensorSpec((self.num_heads * self.head_dim, self.kv_rank), "matrix"),
                "uv": TensorSpec((self.num_heads * self.value_dim, self.kv_rank), "matrix")}

    def bind(self, get):
        self.qdg.bind(get)
        self.out.bind(get)
        self.c_norm = get("dkv.norm")
        self.sink = get("sink").float().contiguous() if self.has_sink else None        # the softmax is float32
        # per head: Wuk_h^T [kv_rank, dim] (the weight of q_h -> its absorbed part) and Wuv_h [vdim, kv_rank] as stored
        self.uk_t = get("uk").view(self.num_heads, self.head_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.uv = get("uv").view(self.num_heads, self.value_dim, self.kv_rank).contiguous()

    def cache_need(self):
        return KvCacheNeed(1, self.row, None, planes=1)

    def __call__(self, x, ctx, cache, residual=None, write_cache=True, out_dtype=None):
        k = ctx.kernels
        meta = ctx.attention[cache.group]
        tables = self.position.rotation_tables() if self.position is not None else None
        cos, sin = tables if tables is not None else (None, None)
        H, R = self.num_heads, self.kv_rank
        proj = self.qdg(x, ctx, out_dtype=torch.float32)          # rounded once, after the norm and the rotation
        q_plain, q_row, gate = k.latent_prepare(proj, self.c_norm, self.eps, ctx.positions, cos, sin, meta.slot_mapping,
                                                cache.kv, H, self.head_dim, self.rot_dim, R, x.dtype,
                                                with_gate=self.has_gate, write_kv=write_cache, halves=self.pairs == "halves")
        k.head_linear(q_plain, self.uk_t, q_row[:, :, :R])        # the absorbed part of every head's query
        o = k.latent_attention(q_row, cache.kv, meta, H, self.row, R, self.scale, gate=gate, sinks=self.sink)     # [T, H, kv_rank]
        o = k.head_linear(o, self.uv, None)                        # [T, H, vdim]
        return self.out(o.view(o.shape[0], H * self.value_dim), ctx, residual=residual, out_dtype=out_dtype)


MIXERS.register("latent_attention", LatentAttention)
