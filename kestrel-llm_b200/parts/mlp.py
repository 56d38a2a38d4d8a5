"""Gated feed-forward: y = W_down (silu(W_gate x) * W_up x), silu(z) = z / (1 + exp(-z))
(reference: st.c:8904-8914, st.c:3605-3607).  Gate and up are one fused product.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import ops
from .base import FeedForward, WeightSlot
from .linear import Linear


class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, width: int, intermediate: int, dtype: torch.dtype, device, prefix: str,
                 activation: str = "silu", names=("gate_proj.weight", "up_proj.weight", "down_proj.weight")):
        if activation != "silu":
            raise ValueError(f"activation '{activation}' has no kernel; only 'silu'")
        self.width, self.intermediate = width, intermediate
        self.prefix, self.names = prefix, names
        self.dtype = dtype
        self.gate_up = Linear(width, 2 * intermediate, dtype, device)
        self.down = Linear(intermediate, width, dtype, device)

    def weight_slots(self) -> List[WeightSlot]:
        p, ff, (gate, up, down) = self.prefix, self.intermediate, self.names
        return [WeightSlot(p + gate, self.gate_up.weight[:ff]),
                WeightSlot(p + up, self.gate_up.weight[ff:]),
                WeightSlot(p + down, self.down.weight)]

    def forward(self, x: torch.Tensor, batch, residual: Optional[torch.Tensor] = None) -> Optional[ops.Partials]:
        act = ops.gate_up_swiglu(x, self.gate_up.weight, self.intermediate, weights_static=True)
        return self.down.forward(act, residual=residual)

    def emit(self, prog, x: int, residual: Optional[int]) -> int:
        act = prog.gate_up_swiglu(x, self.gate_up.weight, self.intermediate)
        return self.down.emit(prog, act, residual=residual, phase="down")


class DenseMLP(FeedForward):
    """Feed-forward without a gate: y = W_down act(W_up x), ``activation`` "relu2" (the square of
    relu), "silu", "tanh", "gelu" (the exact one, with erf) or "gelu_tanh"."""
    graph_safe = True

    def __init__(self, width: int, intermediate: int, dtype: torch.dtype, device, prefix: str, activation: str = "relu2",
                 names=("up", "down")):
        if activation not in ("relu2", "silu", "tanh", "gelu", "gelu_tanh"):
            raise ValueError(f"activation '{activation}' has no kernel; one of 'relu2', 'silu', 'tanh', 'gelu', 'gelu_tanh'")
        self.width, self.intermediate, self.activation = width, intermediate, activation
        self.prefix, self.names, self.dtype = prefix, names, dtype
        self.up = Linear(width, intermediate, dtype, device)
        self.down = Linear(intermediate, width, dtype, device)

    def weight_slots(self) -> List[WeightSlot]:
        return [WeightSlot(self.prefix + self.names[0], self.up.weight), WeightSlot(self.prefix + self.names[1], self.down.weight)]

    def forward(self, x: torch.Tensor, batch) -> ops.Partials:
        # many tokens in bfloat16: the activation is the up product's epilogue; otherwise its slices are summed and activated
        return self.down.forward(ops.linear_act(x, self.up.weight, self.activation, weights_static=True))
