"""Grouped-query attention whose softmax weights are mixed across the heads before they meet the values, over
the paged cache; keys and values may differ in width.

    q = Wq h (+ b), k = Wk h (+ b), v = Wv h (+ b);  v <- v / sqrt(mean(v^2) + eps) per head (option), cached so
    s_h(i, j) = scale q_h(i) . k(j)  -  r1_h ln(1 + r2_h (i - j))                 (option: distance bias)
    visible: j <= i, and with a chunk size C only floor(i / C) = floor(j / C)     (counted from position 0)
    p_h = softmax_j s_h;   p'_h = sum_g talk[h, g] p_g  (option);   o_h = sum_j p'_h(i, j) v_{kv(h)}(j);   y = Wo o (+ b)

No rotation: positions enter through the distance bias and the mask only.  One stacked product gives [q | k | v]
in float32; one kernel rounds q, writes k and the normalised v into the token's cache slot; the attention kernel
forms each head's softmax in float32, mixes the weights of all heads of a token, and applies them.  Scores,
weights, the bias and the mixing matrix are float32.  The cache group is a chunk group: pages below the chunk of
the next query come back while the request runs.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import MIXERS, KvCacheNeed, Part, TensorSpec
from .linear import Linear


class TalkingHeadsAttention(Part):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 value_dim: Optional[int] = None, chunk: Optional[int] = None, value_norm_eps: Optional[float] = None,
                 distance_bias: bool = False, talk: bool = True, bias: bool = False, suffix: str = "", bias_suffix: str = ".b"):
        from ..errors import ConfigError
        value_dim = head_dim if value_dim is None else value_dim
        problems = []
        if num_heads % num_kv_heads:
            problems.append(f"{num_heads} query heads cannot share {num_kv_heads} key/value heads")
        if head_dim > 256 or value_dim > 256:
            problems.append(f"head sizes are at most 256, got {head_dim} and {value_dim}")
        if num_heads > 64:
            problems.append(f"at most 64 heads can exchange their weights, got {num_heads}")
        if chunk is not None and chunk < 1:
            problems.append(f"the chunk size must be positive, got {chunk}")
        if problems:
            raise ConfigError(problems, "talking-heads attention")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.value_dim, self.scale, self.chunk = head_dim, value_dim, float(scale), chunk
        self.value_norm_eps, self.has_distance_bias, self.has_talk = value_norm_eps, distance_bias, talk
        self.q_dim, self.k_dim, self.v_dim = num_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * value_dim
        self.qkv = Linear(hidden_size, [self.q_dim, self.k_dim, self.v_dim], ["q", "k", "v"], bias=bias, suffix=suffix,
                          bias_suffix=bias_suffix)
        self.out = Linear(num_heads * value_dim, [hidden_size], ["o"], bias=bias, suffix=suffix, bias_suffix=bias_suffix)
        self.r1 = self.r2 = self.talk = None

    def tensor_specs(self):
        specs = {**self.qkv.tensor_specs(), **self.out.tensor_specs()}
        if self.has_distance_bias:
            specs["r1"] = TensorSpec((self.num_heads,), "coef")
            specs["r2"] = TensorSpec((self.num_heads,), "coef")
        if self.has_talk:
            specs["talk"] = TensorSpec((self.num_heads, self.num_heads), "mixing")
        return specs

    def bind(self, get):
        self.qkv.bind(get)
        self.out.bind(get)
        if self.has_distance_bias:       # scores and weights are float32
            self.r1, self.r2 = get("r1").float().contiguous(), get("r2").float().contiguous()
        if self.has_talk:
            self.talk = get("talk").float().contiguous()

    def cache_need(self):
        return KvCacheNeed(self.num_kv_heads, self.head_dim, None, 2, self.value_dim, self.chunk)

    def __call__(self, x, ctx, cache, residual=None, write_cache=True, out_dtype=None):
        k = ctx.kernels
        meta = ctx.attention[cache.group]
        proj = self.qkv(x, ctx, out_dtype=torch.float32)
        q = k.kv_prepare(proj, meta.slot_mapping, cache.kv, self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim,
                         self.value_norm_eps, x.dtype, write_kv=write_cache)
        o = k.talking_attention(q, cache.kv, meta, ctx.positions, self.num_heads, self.num_kv_heads, self.head_dim,
                                self.value_dim, self.scale, self.r1, self.r2, self.talk, self.chunk)
        return self.out(o, ctx, residual=residual, out_dtype=out_dtype)


MIXERS.register("talking_heads_attention", TalkingHeadsAttention)
