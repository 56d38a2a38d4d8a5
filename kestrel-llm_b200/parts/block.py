"""Pre-norm residual block: x += mixer(norm1(x)); x += ffn(norm2(x))
(reference: st.c:16412-16413 and 16622-16626 for the attention half, st.c:16704-16705 and
16796-16797 for the feed-forward half).  The output of the feed-forward is handed on unadded,
so that the next block's first norm (or the final norm) adds it while normalising - unless the
part added it to the stream itself (a many-token product does that in its epilogue), in which
case nothing is pending.  A block may be built without feed-forward (and second norm): the mixer's
output is then what is handed on.
"""
from __future__ import annotations

import inspect
from typing import List, Optional

import torch

from ..csrc import ops
from .base import Block, FeedForward, Mixer, Norm, WeightSlot
from .linear import Linear
from .norm import RMSNorm


class PreNormBlock(Block):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm], ffn: Optional[FeedForward], dtype: torch.dtype):
        if (norm2 is None) != (ffn is None):
            raise ValueError("the second norm and the feed-forward come together or not at all")
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self.dtype = dtype
        # parts whose forward takes ``residual`` may add their result to the stream themselves
        self._mixer_adds = "residual" in inspect.signature(mixer.forward).parameters
        self._ffn_adds = ffn is not None and "residual" in inspect.signature(ffn.forward).parameters

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None]

    def weight_slots(self) -> List[WeightSlot]:
        return [s for p in self.parts() for s in p.weight_slots()]

    def forward(self, residual: torch.Tensor, pending, batch, cache):
        n = self.norm1.add_forward(residual, pending, self.dtype)
        a = self.mixer.forward(n, batch, cache, residual=residual) if self._mixer_adds else self.mixer.forward(n, batch, cache)
        if self.ffn is None:
            return residual, a
        n = self.norm2.add_forward(residual, a, self.dtype)            # a is None if the mixer added itself
        f = self.ffn.forward(n, batch, residual=residual) if self._ffn_adds else self.ffn.forward(n, batch)
        return residual, f

    @property
    def emits(self) -> bool:
        return self.ffn is not None and all(getattr(p, "emit", None) is not None for p in self.parts())

    def emit(self, prog, residual: int, pending, cache) -> int:
        """This block's operations in a step program; returns the register of what is still to be
        added to the residual stream (the feed-forward's product)."""
        n = self.norm1.emit(prog, residual, pending, self.dtype)
        a = self.mixer.emit(prog, n, residual if self._mixer_adds else None, cache)
        n = self.norm2.emit(prog, residual, a, self.dtype)
        return self.ffn.emit(prog, n, residual if self._ffn_adds else None)


class ParallelBlock(Block):
    """One norm whose output both sublayers read: h = norm(x); x += mixer(h) + ffn(h); then an
    optional per-layer token input, x += side(x, token).  The feed-forward may be absent; it may also hand
    on two products (routed experts and an expert every token takes), which are added in its order."""

    def __init__(self, norm: Norm, mixer: Mixer, ffn: Optional[FeedForward], side, dtype: torch.dtype):
        self.norm, self.mixer, self.ffn, self.side = norm, mixer, ffn, side
        self.dtype = dtype

    def parts(self):
        return [p for p in (self.norm, self.mixer, self.ffn, self.side) if p is not None]

    def weight_slots(self) -> List[WeightSlot]:
        return [s for p in self.parts() for s in p.weight_slots()]

    def forward(self, residual: torch.Tensor, pending, batch, cache):
        from ..csrc import ops
        h = self.norm.add_forward(residual, pending, self.dtype)
        a = self.mixer.forward(h, batch, cache)
        f = self.ffn.forward(h, batch) if self.ffn is not None else None
        f, f2 = f if isinstance(f, tuple) else (f, None)
        if self.side is None:
            ops.add_two(residual, a, f, None, f2)
            return residual, None
        x = torch.empty(residual.shape, dtype=self.dtype, device=residual.device)
        ops.add_two(residual, a, f, x, f2)
        self.side.add_forward(residual, x, batch)
        return residual, None


class SandwichBlock(Block):
    """A norm in front of each sublayer and another on its result, which may be gated first:

        h = norm1(x);  x += norm1b(mixer(h) * sigmoid(W_g1 h + b_g1))
        h = norm2(x);  x += norm2b(ffn(h)   * sigmoid(W_g2 h + b_g2))

    (``gate1`` / ``gate2`` None: no gate on that sublayer; ``ffn`` None: the first line alone.)  A
    sublayer's gate, second norm and add are one kernel, which also makes the norm that follows
    inside the block; the block adds into the stream itself and hands nothing on."""

    def __init__(self, norm1: RMSNorm, mixer: Mixer, norm1b: RMSNorm, gate1: Optional[Linear], norm2: Optional[RMSNorm],
                 ffn: Optional[FeedForward], norm2b: Optional[RMSNorm], gate2: Optional[Linear], dtype: torch.dtype, prefix: str,
                 gate_names=("rg1", "rg2")):
        if len({norm2 is None, ffn is None, norm2b is None}) != 1:
            raise ValueError("the feed-forward comes with both of its norms or not at all")
        if ffn is None and gate2 is not None:
            raise ValueError("a gate for a feed-forward that is not there")
        self.norm1, self.mixer, self.norm1b, self.gate1 = norm1, mixer, norm1b, gate1
        self.norm2, self.ffn, self.norm2b, self.gate2 = norm2, ffn, norm2b, gate2
        self.dtype, self.prefix, self.gate_names = dtype, prefix, gate_names

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm1b, self.norm2, self.ffn, self.norm2b) if p is not None]

    def weight_slots(self) -> List[WeightSlot]:
        slots = [s for p in self.parts() for s in p.weight_slots()]
        for gate, name in zip((self.gate1, self.gate2), self.gate_names):
            if gate is not None:
                slots.append(WeightSlot(self.prefix + name, gate.weight))
                if gate.bias is not None:
                    slots.append(WeightSlot(self.prefix + name + ".b", gate.bias, "bias"))
        return slots

    def forward(self, residual: torch.Tensor, pending, batch, cache):
        h = self.norm1.add_forward(residual, pending, self.dtype)
        y = self.mixer.forward(h, batch, cache)
        g = self.gate1.forward(h) if self.gate1 is not None else None
        if self.ffn is None:
            ops.add_gated_normed(residual, y, g, self.norm1b.weight, self.norm1b.eps)
            return residual, None
        h = torch.empty(residual.shape, dtype=self.dtype, device=residual.device)
        ops.add_gated_normed(residual, y, g, self.norm1b.weight, self.norm1b.eps, self.norm2.weight, self.norm2.eps, h)
        z = self.ffn.forward(h, batch)
        g = self.gate2.forward(h) if self.gate2 is not None else None
        ops.add_gated_normed(residual, z, g, self.norm2b.weight, self.norm2b.eps)
        return residual, None
