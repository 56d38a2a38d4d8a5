"""Token embedding and the output head.

x = E[token] widened to float32 (st.c:16392-16393); logits = W_lm n in float32
(st.c:16850-16855).  A tied head shares the embedding's memory
(vqf_convert/src/conv_main.c:613-614).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import ops
from .base import Part, WeightSlot


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab: int, width: int, dtype: torch.dtype, device, weight_name: str, scale: float = 1.0):
        self.vocab, self.width = vocab, width
        self.weight = torch.empty((vocab, width), dtype=dtype, device=device)
        self.weight_name = weight_name
        self.scale = float(scale)              # x = E[token] * scale
        if self.scale != 1.0:
            self.emit = None                   # the step program's embedding has no factor: such a model walks its parts

    def weight_slots(self) -> List[WeightSlot]:
        return [WeightSlot(self.weight_name, self.weight)]

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        out = torch.empty((token_ids.shape[0], self.width), dtype=torch.float32, device=token_ids.device)
        ops.embed(self.weight, token_ids, out, self.scale)
        return out

    def add_forward(self, token_ids: torch.Tensor, x: torch.Tensor) -> None:
        """x += E[token]: the embedded tokens fed into the stream once more."""
        ops.embed_add(self.weight, token_ids, x)

    def emit(self, prog) -> int:
        return prog.embed(self.weight)


class StreamRows(Part):
    """Learned vectors of the stream's width, one of which is added to every token of the stream in front of a
    layer call (`LayerCall.add_row`): float32 [rows, width]."""
    graph_safe = True

    def __init__(self, rows: int, width: int, device, weight_name: str):
        self.weight = torch.empty((rows, width), dtype=torch.float32, device=device)
        self.weight_name = weight_name

    def weight_slots(self) -> List[WeightSlot]:
        return [WeightSlot(self.weight_name, self.weight, "bias")]

    def add_forward(self, row: int, x: torch.Tensor) -> None:
        ops.add_row(x, self.weight[row])


class LMHead(Part):
    """``scale`` multiplies the logits; ``softcap`` > 0 then bounds them, cap * tanh(logits / cap)."""
    graph_safe = True

    def __init__(self, vocab: int, width: int, dtype: torch.dtype, device, weight_name: str,
                 tied_to: Optional[TokenEmbedding] = None, scale: float = 1.0, softcap: float = 0.0):
        self.vocab, self.width = vocab, width
        self.weight_name = weight_name
        self.scale, self.softcap = float(scale), float(softcap)
        if self.softcap < 0:
            raise ValueError("a cap on the logits is positive, or 0 for none")
        self.plain = self.scale == 1.0 and self.softcap == 0.0     # the product alone: what a step program's output head does
        self.tied = tied_to is not None
        self.weight = tied_to.weight if tied_to is not None else \
            torch.empty((vocab, width), dtype=dtype, device=device)

    def weight_slots(self) -> List[WeightSlot]:
        return [] if self.tied else [WeightSlot(self.weight_name, self.weight)]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [R, width] -> float32 logits [R, vocab].  The product is not split over K (a split
        product returns slices that a consumer kernel sums; the logits have no such consumer)."""
        logits = torch.empty((1, x.shape[0], self.vocab), dtype=torch.float32, device=x.device)
        logits = ops.linear(x, self.weight, logits, weights_static=True)[0]
        if not self.plain:
            ops.logit_scale_cap(logits, self.scale, self.softcap)
        return logits

    def emit(self, prog, x: int) -> None:
        prog.logits(x, self.weight)
