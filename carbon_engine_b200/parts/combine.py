"""Mixers side by side: several mixers read the same input and their outputs are added with fixed weights,

    y = sum_i weight_i mixer_i(h)

Each member keeps a cache of its own kind (pages, a state, a bundle); the layer's cache is a bundle of them, and every
member sees the view it would see alone.  A member's weight becomes its ``out_scale`` (it multiplies the heads' outputs in
the kernel that stores them, before the member's output product adds into the residual), so a member must have one.
"""
from __future__ import annotations

from typing import Any, List, Sequence, Tuple

import torch

from ..cache.storage import LayerCacheView
from .base import BundleCacheSpec, Mixer, PagedCacheSpec, Part, StateCacheSpec


class SummedMixers(Mixer):
    can_store = True

    def __init__(self, members: Sequence[Mixer], weights: Sequence[float]):
        if len(members) != len(weights) or not members:
            raise ValueError("one weight per mixer")
        for m in members:
            if not hasattr(m, "out_scale"):
                raise ValueError(f"{type(m).__name__} has no out_scale and cannot be weighted in a sum of mixers")
            if not getattr(m, "can_store", False):
                raise ValueError(f"{type(m).__name__} cannot store its output")
        self.members, self.weights = list(members), [float(w) for w in weights]
        for m, w in zip(self.members, self.weights):
            m.out_scale = w
        # where each member's cache lives in the layer's bundle: the one paged cache (or else the first state) is the
        # bundle's main cache, every other state an extra named after the member
        specs = [m.cache_spec() for m in self.members]
        mains = [s.main if isinstance(s, BundleCacheSpec) else s for s in specs]
        paged = [i for i, s in enumerate(mains) if isinstance(s, PagedCacheSpec)]
        if len(paged) > 1:
            raise ValueError("at most one of the mixers may keep keys and values in pages")
        states = [i for i, s in enumerate(mains) if isinstance(s, StateCacheSpec)]
        self._main = paged[0] if paged else (states[0] if states else -1)
        extra: List[Tuple[str, StateCacheSpec]] = []
        for i, s in enumerate(specs):
            if i != self._main and isinstance(mains[i], StateCacheSpec):
                extra.append((f"{i}.state", mains[i]))
            if isinstance(s, BundleCacheSpec):
                extra += [(f"{i}.{name}", st) for name, st in s.extra]
        self._spec = BundleCacheSpec(mains[self._main] if self._main >= 0 else None, tuple(extra)) if extra else \
            (mains[self._main] if self._main >= 0 else None)

    @property
    def graph_safe(self) -> bool:
        return all(getattr(m, "graph_safe", False) for m in self.members)

    def children(self) -> List[Part]:
        return list(self.members)

    def planners(self) -> List[Mixer]:
        return [p for m in self.members for p in m.planners()]

    def cache_spec(self):
        return self._spec

    def step_bytes(self, tokens: int, element_size: int) -> int:
        return max(m.step_bytes(tokens, element_size) for m in self.members)

    def _view(self, i: int, cache) -> Any:
        """What member ``i`` would see of a cache of its own."""
        extra = {name[len(f"{i}."):]: t for name, t in (cache.extra or {}).items() if name.startswith(f"{i}.")}
        if i == self._main:
            return LayerCacheView(cache.kind, cache.group, cache.page_size, cache.k_pool, cache.v_pool, cache.state, cache.writes,
                                  extra or None)
        state = extra.pop("state", None)
        return LayerCacheView("state" if state is not None else "none", state=state, writes=cache.writes, extra=extra or None)

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor, cache, accumulate: bool = True) -> None:
        for i, m in enumerate(self.members):
            # the first member stores where the caller wants a stored result; the others add to it
            m.forward(ctx, h, x, self._view(i, cache), accumulate=accumulate or i > 0)
