"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from parameters only (sizes and constants; never a model's name), says which
tensors it owns (`tensor_specs`, names relative to its prefix) and receives them through
`bind`.  Kinds of part and what each must offer:

* position encoding: `prepare(max_len, device)`; `rotation_tables()` -> (cos, sin) float
  tables [max_len, rotary_dim/2] or None; `on_embeddings(x, ctx)` -> x for encodings that act
  on the input of the first layer.
* norm: `__call__(x, ctx)` -> tensor of the same shape.
* mixer: `cache_need()` -> `KvCacheNeed`, `StateNeed`, `CompositeNeed` (several of these, for a mixer
  made of mixers) or None;
  `__call__(x, ctx, cache, residual, write_cache)` -> residual + mixed x.  `cache` is the
  `CacheView` of the run entry's cache slot (with one sub-view per member of a `CompositeNeed`).
* feed-forward: `__call__(x, ctx, residual)` -> residual + f(x).
* block: built from `parts`, the layer's built parts by role name (which roles it needs is the
  block's own matter), plus its parameters; `__call__(x, ctx, cache, write_cache)` -> x.
* hook: `__call__(x, ctx)` -> x, on the embedded tokens or on the float32 logits.

A part whose step cannot be recorded into a CUDA graph (it reads device values on the host, or
launches a number of kernels that depends on the data) sets `graph_safe = False`; a model with
such a part runs its decode steps eagerly.

`ctx` is the step's `StepContext` (tokens' positions, the attention metadata of each cache
group, state slots, the kernel library).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class TensorSpec:
    shape: Tuple[int, ...]
    init: str          # "matrix", "norm" or "bias": which random distribution fills it


@dataclass(frozen=True)
class KvCacheNeed:
    """Paged keys and values; `window` None keeps every key, W keeps the last W.  `planes` is 2 for
    separate key and value rows, 1 for mixers that keep ONE row per token and head from which both are
    read (a latent that keys and values are projections of).  `value_dim`: the size of a value row where it
    differs from the key's `head_dim` (a page then holds all its key rows followed by all its value rows,
    and the group's tensor is flat per page).  `chunk` C: a query at position i reads keys of its own block of
    C positions only (floor(i / C) = floor(j / C)), so pages that lie wholly below the block of the next
    query are given back."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    planes: int = 2
    value_dim: Optional[int] = None
    chunk: Optional[int] = None

    @property
    def row_elements(self) -> int:
        """Elements one token keeps per kv head over all planes."""
        if self.value_dim is None or self.planes != 2:
            return self.planes * self.head_dim
        return self.head_dim + self.value_dim

    @property
    def flat_pages(self) -> bool:
        return self.planes == 2 and self.value_dim is not None and self.value_dim != self.head_dim


@dataclass(frozen=True)
class StateNeed:
    """State of fixed size per request (shape without the request dimension)."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclass(frozen=True)
class CompositeNeed:
    """What a mixer made of several mixers needs: one entry per member (`KvCacheNeed`, `StateNeed` or None), in
    the members' order.  The run entry's `CacheView` then carries one sub-view per member in `parts`."""
    parts: Tuple[object, ...]


class Part:
    graph_safe = True      # whether the part's work in a decode step may be captured in a CUDA graph

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        """`get(name)` returns the device tensor stored under the part's prefix + name."""


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: Dict[str, Callable[..., Any]] = {}

    def register(self, kind: str, factory: Callable[..., Any]) -> None:
        self._items[kind] = factory

    def unregister(self, kind: str) -> None:
        self._items.pop(kind, None)

    def build(self, kind: str, **params):
        if kind not in self._items:
            from ..errors import ConfigError
            raise ConfigError(f"unknown {self.what} {kind!r}; known: {', '.join(sorted(self._items))}")
        return self._items[kind](**params)

    def known(self):
        return sorted(self._items)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block arrangement")
HOOKS = Registry("hook")
FAMILIES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS}
