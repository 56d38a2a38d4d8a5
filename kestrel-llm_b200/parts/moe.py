"""Routed feed-forward: E small gated experts, of which each token uses ``top``.

Router logits z = W_r h + b in float32; the ``top`` largest are chosen and weighted by the
softmax over the chosen logits alone.  An expert with a clamp ``limit``:

    g = min(W_gate h, limit);  u = clamp(W_up h, -limit, limit);  y = W_down (g sigmoid(1.702 g) (u + 1))

The experts' matrices are stacked ([E, 2 ff, width] gate rows then up rows, [E, width, ff]), the
step's (token, choice) pairs are grouped by expert on the device, and two grouped products run
them; a token's result does not depend on the batch.

`GroupRoutedExperts` is a routed feed-forward of another kind: experts without a gate, y = W_down act(W_up h) with
``activation`` a parameter and no biases; a router whose scores are s = sigmoid(W_r h) in float32, which CHOOSES by
s + correction[e] (a learned number per expert) but weighs by s alone; experts in ``groups`` equal groups of neighbours, a
group's score the sum of its two largest choice scores, only experts of the ``keep`` best groups open to choice (the
others count as minus infinity); weights = the chosen experts' s over their sum (+ 1e-20) times ``scale``; and optionally
one more expert of the same form that every token takes (``shared_inner`` > 0), whose product is handed on beside the
routed experts' so that the block adds both.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import ops
from .base import FeedForward, WeightSlot
from .linear import Linear
from .mlp import DenseMLP


class RoutedExperts(FeedForward):
    graph_safe = True          # forward launches kernels over device tensors of the batch only

    def __init__(self, width: int, inner: int, experts: int, top: int, limit: float, dtype: torch.dtype, device, prefix: str,
                 router_bias: bool = True, expert_name: str = "e{}."):
        if not 1 <= top <= min(experts, 32):
            raise ValueError(f"top = {top} of {experts} experts: the router kernel takes 1 to min(experts, 32)")
        self.width, self.inner, self.experts, self.top, self.limit = width, inner, experts, top, float(limit)
        self.dtype, self.prefix, self.expert_name = dtype, prefix, expert_name
        self.router = Linear(width, experts, dtype, device)
        self.router_bias: Optional[torch.Tensor] = torch.empty((experts,), dtype=torch.float32, device=device) if router_bias else None
        self.w_gate_up = torch.empty((experts, 2 * inner, width), dtype=dtype, device=device)
        self.w_down = torch.empty((experts, width, inner), dtype=dtype, device=device)

    def weight_slots(self) -> List[WeightSlot]:
        p, ff = self.prefix, self.inner
        slots = [WeightSlot(p + "router", self.router.weight)]
        if self.router_bias is not None:
            slots.append(WeightSlot(p + "router.b", self.router_bias, "bias"))
        for e in range(self.experts):
            q = p + self.expert_name.format(e)
            slots += [WeightSlot(q + "gate", self.w_gate_up[e, :ff]), WeightSlot(q + "up", self.w_gate_up[e, ff:]),
                      WeightSlot(q + "down", self.w_down[e])]
        return slots

    def forward(self, x: torch.Tensor, batch) -> ops.Partials:
        ids, weights = ops.moe_route(self.router.forward(x), self.router_bias, self.top)
        return ops.Partials(ops.moe_experts(x, ids, weights, self.w_gate_up, self.w_down, self.limit))


class GroupRoutedExperts(FeedForward):
    graph_safe = True          # forward launches kernels over device tensors of the batch only

    def __init__(self, width: int, inner: int, experts: int, top: int, dtype: torch.dtype, device, prefix: str, groups: int = 1,
                 keep: int = 1, scale: float = 1.0, activation: str = "gelu", shared_inner: int = 0, correction: bool = True,
                 expert_name: str = "e{}.", names=("up", "down", "router", "correction", "shared.")):
        if not 1 <= top <= min(experts, 32):
            raise ValueError(f"top = {top} of {experts} experts: the router kernel takes 1 to min(experts, 32)")
        if experts % groups or not 1 <= keep <= groups or top > keep * (experts // groups):
            raise ValueError(f"{experts} experts in {groups} groups, {keep} kept, {top} chosen do not fit")
        if activation not in ops.UP_ACTS:
            raise ValueError(f"activation '{activation}' has no kernel; one of {', '.join(ops.UP_ACTS)}")
        self.width, self.inner, self.experts, self.top = width, inner, experts, top
        self.groups, self.keep, self.scale, self.activation = groups, keep, float(scale), activation
        self.dtype, self.prefix, self.expert_name, self.names = dtype, prefix, expert_name, names
        self.router = Linear(width, experts, dtype, device)
        self.correction: Optional[torch.Tensor] = torch.empty((experts,), dtype=torch.float32, device=device) if correction else None
        self.w_up = torch.empty((experts, inner, width), dtype=dtype, device=device)
        self.w_down = torch.empty((experts, width, inner), dtype=dtype, device=device)
        self.shared = DenseMLP(width, shared_inner, dtype, device, prefix + names[4], activation=activation, names=names[:2]) \
            if shared_inner else None

    def weight_slots(self) -> List[WeightSlot]:
        p, (up, down, router, correction, _shared) = self.prefix, self.names
        slots = [WeightSlot(p + router, self.router.weight)]
        if self.correction is not None:
            slots.append(WeightSlot(p + correction, self.correction, "bias"))
        for e in range(self.experts):
            q = p + self.expert_name.format(e)
            slots += [WeightSlot(q + up, self.w_up[e]), WeightSlot(q + down, self.w_down[e])]
        if self.shared is not None:
            slots += self.shared.weight_slots()
        return slots

    def forward(self, x: torch.Tensor, batch):
        """The routed experts' product, or (routed, shared) where every token also takes the shared expert."""
        ids, weights = ops.moe_route_sigmoid(self.router.forward(x), self.correction, self.top, self.groups, self.keep, self.scale)
        routed = ops.Partials(ops.moe_experts_ungated(x, ids, weights, self.w_up, self.w_down, self.activation).unsqueeze(0))
        if self.shared is None:
            return routed
        return routed, self.shared.forward(x, batch)
