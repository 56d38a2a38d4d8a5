"""A recurrent mixer with a real-gated linear recurrent unit (the recurrent block of the Griffin family of
models): two branches of C channels off the mixer's input h, one a gate, one a diagonal recurrence whose decay
and input gate are made from the recurrence's own input.

    y = gelu_tanh(W_y h + b_y)
    u = conv(W_x h + b_x) + b_conv              causal convolution over time per channel, `taps` wide, zeros before the start
    r = sigmoid(Wa_b u_b + ba),  i = sigmoid(Wi_b u_b + bi)     per block b of C / blocks channels: block-diagonal products
    a = exp(-rate * r * softplus(lam))          per channel
    S <- a S + sqrt(1 - a^2) * (i * u)          S starts at zero; the first token is no special case
    out = W_o (S * y)

W_y and W_x are one fused product.  The state S and the convolution's last taps - 1 inputs live in the request's state
slot, in float32; decays, gates, softplus, exponentials and the recurrence are float32 in every mode; the gates'
block-diagonal products are head-wise products (`ops.head_gemm`) with float32 results.  ``rate`` is the constant in the
decay's exponent (8 in the published design).
"""
from __future__ import annotations

from typing import List

import torch

from ..csrc import ops
from .base import FixedStateSpec, Mixer, WeightSlot
from .linear import Linear


class GatedDiagonalRecurrence(Mixer):
    graph_safe = True          # forward launches kernels over device tensors of the batch only

    def __init__(self, width: int, channels: int, blocks: int, taps: int, dtype: torch.dtype, device, prefix: str, rate: float = 8.0,
                 names=("y", "x", "conv", "ra", "ri", "lam", "o")):
        if channels % blocks:
            raise ValueError(f"{channels} channels do not divide into {blocks} blocks")
        if not 1 <= taps <= 9:
            raise ValueError(f"{taps} taps: the convolution kernel takes 1 to 9")
        self.width, self.C, self.blocks, self.taps, self.rate = width, channels, blocks, taps, float(rate)
        self.dtype, self.prefix, self.names = dtype, prefix, names
        bw = channels // blocks
        f32 = dict(dtype=torch.float32, device=device)
        self.in_proj = Linear(width, 2 * channels, dtype, device, bias=True)         # columns [y | x]
        self.out = Linear(channels, width, dtype, device)
        self.conv_w = torch.empty((channels, taps), **f32)
        self.conv_b = torch.empty((channels,), **f32)
        self.w_r = torch.empty((blocks * bw, bw), dtype=dtype, device=device)          # block b's matrix [out, in] in rows b bw ..
        self.w_i = torch.empty((blocks * bw, bw), dtype=dtype, device=device)
        self.b_r = torch.empty((channels,), **f32)
        self.b_i = torch.empty((channels,), **f32)
        self.lam = torch.empty((channels,), **f32)
        self.tail_off = channels                                # the slot: S [C], then the convolution's tail [taps - 1, C]
        self.state_size = channels * taps

    def cache_spec(self) -> FixedStateSpec:
        return FixedStateSpec((self.state_size,), torch.float32)

    def weight_slots(self) -> List[WeightSlot]:
        p, (y, x, conv, ra, ri, lam, o), C = self.prefix, self.names, self.C
        bw = C // self.blocks
        w, b = self.in_proj.weight, self.in_proj.bias
        return [WeightSlot(p + y, w[:C]), WeightSlot(p + y + ".b", b[:C], "bias"), WeightSlot(p + x, w[C:]), WeightSlot(p + x + ".b", b[C:], "bias"),
                WeightSlot(p + conv, self.conv_w), WeightSlot(p + conv + ".b", self.conv_b, "bias"),
                WeightSlot(p + ra, self.w_r.view(self.blocks, bw, bw)), WeightSlot(p + ra + ".b", self.b_r.view(self.blocks, bw), "bias"),
                WeightSlot(p + ri, self.w_i.view(self.blocks, bw, bw)), WeightSlot(p + ri + ".b", self.b_i.view(self.blocks, bw), "bias"),
                WeightSlot(p + lam, self.lam, "bias"), WeightSlot(p + o, self.out.weight)]

    def forward(self, x: torch.Tensor, batch, cache) -> ops.Partials:
        T, dev, f32, C = x.shape[0], x.device, torch.float32, self.C
        fused = self.in_proj.forward(x)
        y = torch.empty((T, C), dtype=f32, device=dev)
        u = torch.empty((T, C), dtype=f32, device=dev)
        u_st = torch.empty((T, C), dtype=self.dtype, device=dev)
        ops.rglru_branches(fused, self.conv_w, self.conv_b, cache.state, self.tail_off, batch, y, u, u_st)
        gr = ops.head_gemm(u_st, self.w_r, self.blocks, w_kn=False, out_f32=True)
        gi = ops.head_gemm(u_st, self.w_i, self.blocks, w_kn=False, out_f32=True)
        out = torch.empty((T, C), dtype=self.dtype, device=dev)
        ops.rglru_scan(y, u, gr, gi, self.b_r, self.b_i, self.lam, self.rate, cache.state, batch, out)
        return self.out.forward(out)
