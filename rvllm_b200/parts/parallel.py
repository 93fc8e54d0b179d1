"""Several mixers side by side: each reads the same input, the result is the weighted sum of theirs.

    y = sum_b scale_b * mixer_b(h)

`branches` lists the members: {"kind": registry key, "params": {...}, "prefix": tensor sub-prefix, "scale": number}.
Every member keeps its own cache or state: the part's need is a `CompositeNeed` with one entry per member, and the
run entry's cache view carries one sub-view per member.  The members return float32 and the sum is float32.
"""
from __future__ import annotations

import torch

from .base import MIXERS, CompositeNeed, Part


class ParallelMixers(Part):
    def __init__(self, branches, position=None):
        from ..errors import ConfigError
        if not branches:
            raise ConfigError("a parallel mixer needs at least one member")
        self.members, self.prefixes, self.scales = [], [], []
        for b in branches:
            params = dict(b.get("params", {}))
            self.members.append(MIXERS.build(b["kind"], **params))
            self.prefixes.append(b.get("prefix", ""))
            self.scales.append(float(b.get("scale", 1.0)))
        if len(set(self.prefixes)) != len(self.prefixes):
            raise ConfigError(f"the members of a parallel mixer need distinct tensor prefixes, got {self.prefixes}")

    @property
    def graph_safe(self):
        return all(getattr(m, "graph_safe", True) for m in self.members)

    def tensor_specs(self):
        return {p + name: ts for m, p in zip(self.members, self.prefixes) for name, ts in m.tensor_specs().items()}

    def bind(self, get):
        for m, p in zip(self.members, self.prefixes):
            m.bind(lambda name, _p=p: get(_p + name))

    def cache_need(self):
        return CompositeNeed(tuple(m.cache_need() for m in self.members))

    def __call__(self, x, ctx, cache, residual=None, write_cache=True, out_dtype=None):
        k = ctx.kernels
        total = None
        for m, view, scale in zip(self.members, cache.parts, self.scales):
            y = m(x, ctx, view, residual=None, write_cache=write_cache, out_dtype=torch.float32)
            total = k.scaled_sum(total, 1.0, y, scale)
        if residual is not None:
            total = k.scaled_sum(total, 1.0, residual if residual.dtype == torch.float32 else residual.float(), 1.0)
        return total if out_dtype in (None, torch.float32) else total.to(out_dtype)


MIXERS.register("parallel_mixers", ParallelMixers)
