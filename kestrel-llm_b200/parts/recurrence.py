"""Recurrent mixers whose memory is a matrix per head, carried from token to token in the
request's state slot (float32, zero at admission).  Both run on one scan,

    S_t = diag(w_t) S_{t-1} + a_t (b_t^T S_{t-1}) + k_t v_t^T,      o_t = S_t^T r_t        (`ops.recurrence_scan`)

with everything that enters it in float32; what differs is how a layer makes w, a, b, k, v, r
from its input h.

`ForgetGateRecurrence` (the HGRN2 form of linear attention): H heads, d key and dv value channels,

    r = silu(W_q h),  v = W_v h,  f = lower + (1 - lower) * sigmoid(W_f h + b_f),  w = f,  k = 1 - f

(no correction term: the forget gate alone decides what stays and what is written), then each head's
o is RMS-normed over dv with ONE weight [dv] that the heads share, and projected by W_o.

`RemovalDeltaMixer` (a generalised delta rule): H heads of d key and d value channels,

    r, k, v = W_r h, W_k h, W_v h;   u = k / sqrt(sum k^2 + 1e-6) per head
    w = exp(-decay_rate * sigmoid(W_w2 tanh(W_w1 h) + w0)),   rate = sigmoid(W_a h + b_a)
    a = -(rate * u),  b = u

(what the old state holds along the unit key leaves it at `rate` per channel, beside the decay and
before the write), then each head's o is divided by its root mean square, the heads are multiplied
by a weight [H d] and by sigmoid(W_g h), and projected by W_o.  ``decay_rate`` is a constant of the
design that uses the mixer.
"""
from __future__ import annotations

from typing import List

import torch

from ..csrc import ops
from .base import FixedStateSpec, Mixer, WeightSlot
from .linear import Linear


class ForgetGateRecurrence(Mixer):
    graph_safe = True          # forward launches kernels over device tensors of the batch only

    def __init__(self, width: int, heads: int, key_dim: int, value_dim: int, norm_eps: float, dtype: torch.dtype, device, prefix: str,
                 names=("q", "f", "v", "o", "lower", "norm")):
        if key_dim > 256:
            raise ValueError(f"key size {key_dim}: the scan holds up to 256 key channels a column")
        self.width, self.H, self.d, self.dv = width, heads, key_dim, value_dim
        self.eps, self.dtype, self.prefix, self.names = float(norm_eps), dtype, prefix, names
        n, nv = heads * key_dim, heads * value_dim
        self.col_q, self.col_f, self.col_v = 0, n, 2 * n
        self.in_proj = Linear(width, 2 * n + nv, dtype, device)
        self.out = Linear(nv, width, dtype, device)
        f32 = dict(dtype=torch.float32, device=device)
        self.f_bias = torch.empty((n,), **f32)
        self.lower = torch.empty((n,), **f32)
        self.norm_w = torch.empty((value_dim,), **f32)
        self.state_size = heads * key_dim * value_dim

    def cache_spec(self) -> FixedStateSpec:
        return FixedStateSpec((self.state_size,), torch.float32)

    def weight_slots(self) -> List[WeightSlot]:
        p, w, n = self.prefix, self.in_proj.weight, self.H * self.d
        q, f, v, o, lower, norm = self.names
        return [WeightSlot(p + q, w[:n]), WeightSlot(p + f, w[n:2 * n]), WeightSlot(p + v, w[2 * n:]), WeightSlot(p + o, self.out.weight),
                WeightSlot(p + f + ".b", self.f_bias, "bias"), WeightSlot(p + lower, self.lower, "unit"),
                WeightSlot(p + norm, self.norm_w, "norm")]

    def forward(self, x: torch.Tensor, batch, cache) -> ops.Partials:
        H, d, dv = self.H, self.d, self.dv
        fused = self.in_proj.forward(x)
        r, w, k, v = ops.forget_gates(fused, self.col_q, self.col_f, self.col_v, self.f_bias, self.lower, H * d, H * dv)
        o = ops.recurrence_scan(r, w, k, v, None, None, cache.state, 0, batch, H, d, dv)
        y = torch.empty((x.shape[0], H * dv), dtype=self.dtype, device=x.device)
        ops.head_norm_gate(o, self.norm_w, self.eps, None, 0, y, H, dv)
        return self.out.forward(y)


class RemovalDeltaMixer(Mixer):
    graph_safe = True

    def __init__(self, width: int, heads: int, dim: int, decay_rank: int, decay_rate: float, norm_eps: float, dtype: torch.dtype, device,
                 prefix: str):
        if dim > 256:
            raise ValueError(f"key size {dim}: the scan holds up to 256 key channels a column")
        if decay_rank <= 0:
            raise ValueError("the rank of the decay's two-step projection must be positive")
        self.width, self.H, self.d, self.rank = width, heads, dim, decay_rank
        self.decay_rate, self.eps, self.dtype, self.prefix = float(decay_rate), float(norm_eps), dtype, prefix
        n = heads * dim
        # one product for everything that reads h: r | k | v | rate logits | output gate logits | the decay's first step
        self.col_r, self.col_k, self.col_v, self.col_a, self.col_g, self.col_w1 = 0, n, 2 * n, 3 * n, 4 * n, 5 * n
        self.in_proj = Linear(width, 5 * n + decay_rank, dtype, device)
        self.w2 = Linear(decay_rank, n, dtype, device)
        self.out = Linear(n, width, dtype, device)
        f32 = dict(dtype=torch.float32, device=device)
        self.a_bias = torch.empty((n,), **f32)
        self.w0 = torch.empty((n,), **f32)
        self.norm_w = torch.empty((n,), **f32)
        self.state_size = heads * dim * dim

    def cache_spec(self) -> FixedStateSpec:
        return FixedStateSpec((self.state_size,), torch.float32)

    def weight_slots(self) -> List[WeightSlot]:
        p, w, n = self.prefix, self.in_proj.weight, self.H * self.d
        return [WeightSlot(p + "r", w[:n]), WeightSlot(p + "k", w[n:2 * n]), WeightSlot(p + "v", w[2 * n:3 * n]),
                WeightSlot(p + "a", w[3 * n:4 * n]), WeightSlot(p + "g", w[4 * n:5 * n]), WeightSlot(p + "w1", w[5 * n:]),
                WeightSlot(p + "w2", self.w2.weight), WeightSlot(p + "o", self.out.weight), WeightSlot(p + "a.b", self.a_bias, "bias"),
                WeightSlot(p + "w0", self.w0, "bias"), WeightSlot(p + "norm", self.norm_w, "norm")]

    def forward(self, x: torch.Tensor, batch, cache) -> ops.Partials:
        H, d = self.H, self.d
        fused = self.in_proj.forward(x)
        wz = self.w2.forward(ops.partial_columns_act(fused, self.col_w1, self.rank, self.dtype, "tanh"))
        r, w, k, v, a, b = ops.removal_gates(fused, self.col_r, self.col_k, self.col_v, self.col_a, self.a_bias, wz, self.w0, self.decay_rate,
                                             H, d)
        o = ops.recurrence_scan(r, w, k, v, a, b, cache.state, 0, batch, H, d, d)
        y = torch.empty((x.shape[0], H * d), dtype=self.dtype, device=x.device)
        ops.head_norm_gate(o, self.norm_w, self.eps, fused, self.col_g, y, H, d)
        return self.out.forward(y)
