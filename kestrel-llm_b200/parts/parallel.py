"""Two mixers side by side on the same input: each one's output is RMS-normed over the model
width with a weight of its own, and the mixer's result is their weighted sum,

    y = mix * (rmsnorm(left(h)) * w_left + rmsnorm(right(h)) * w_right)          (mix = 1/2: the mean)

The two keep what they keep - pages of keys and values, a state slot - in ONE cache layer: its
spec is a `CombinedSpec` of theirs, and both are handed the layer's `LayerCache`, of which each
uses its own part.
"""
from __future__ import annotations

from typing import List

import torch

from ..csrc import ops
from .base import CacheSpec, CombinedSpec, FixedStateSpec, Mixer, PagedKVSpec, WeightSlot


class ParallelMixers(Mixer):
    def __init__(self, left: Mixer, right: Mixer, width: int, norm_eps: float, device, prefix: str, names=("left.out", "right.out"),
                 mix: float = 0.5):
        self.left, self.right, self.width = left, right, width
        self.eps, self.mix, self.prefix, self.names = float(norm_eps), float(mix), prefix, names
        self.w_left = torch.empty((width,), dtype=torch.float32, device=device)
        self.w_right = torch.empty((width,), dtype=torch.float32, device=device)
        specs = [sp for sp in (left.cache_spec(), right.cache_spec()) if sp is not None]
        paged = [sp for sp in specs if isinstance(sp, PagedKVSpec)]
        state = [sp for sp in specs if isinstance(sp, FixedStateSpec)]
        if len(paged) > 1 or len(state) > 1 or len(paged) + len(state) != len(specs):
            raise ValueError("two mixers side by side share one cache layer: at most one of them keeps pages and at most one a state")
        self._spec: CacheSpec = specs[0] if len(specs) == 1 else (CombinedSpec(paged[0], state[0]) if specs else None)

    @property
    def graph_safe(self) -> bool:
        return bool(getattr(self.left, "graph_safe", False) and getattr(self.right, "graph_safe", False))

    def cache_spec(self) -> CacheSpec:
        return self._spec

    def weight_slots(self) -> List[WeightSlot]:
        return self.left.weight_slots() + self.right.weight_slots() + [WeightSlot(self.prefix + self.names[0], self.w_left, "norm"),
                                                                      WeightSlot(self.prefix + self.names[1], self.w_right, "norm")]

    def forward(self, x: torch.Tensor, batch, cache) -> ops.Partials:
        a = self.left.forward(x, batch, cache)
        b = self.right.forward(x, batch, cache)
        for p in (a, b):
            if p.bias is not None:
                raise ValueError("a mixer that runs beside another hands over its product without a pending bias")
        return ops.combine_normed(a, self.w_left, b, self.w_right, self.eps, self.mix)
