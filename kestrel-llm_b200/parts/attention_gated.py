"""Grouped-query softmax attention over a window that keeps the first tokens of a request, with
values of their own size and a gate on every head's output; without rotation unless it is given a
position encoding.

q, k, v and the gate logits are one fused product of the mixer's input h.  q and k are divided by
their root mean square per head (no weight); score = q . k * scale with ``scale`` a parameter;
query i sees key j <= i if i - j < window or j < keep_first (window 0: every j <= i); the output
of head n is multiplied by sigmoid(gate logit n) before the output projection.  K (after the
norm) and V go to the request's pages; a mixer built with ``own_kv=False`` has no key and value
projections and attends over the pages that an earlier layer of the same step wrote, with its
own queries, mask and scale.

Every one of these is a parameter, and there are more, all off by default: biases on the four
projections (``bias``); the norm of q and k taken over the whole projection instead of per head,
with a weight per column (``qk_norm="projection"``), or none at all (``qk_norm=None``); values of unit
root mean square per head, cached so (``v_norm``); a cap on the scores, s <- cap * tanh(s / cap)
(``softcap``); a distance term s <- s - r1[n] * ln(1 + r2[n] * (i - j)) with two numbers per head
(``distance_bias``); and the way keys are weighed (``weighting``): "softmax", "softmax_sink" (the
denominator has one more term that carries no value: exp(0), or exp(sink[n]) with a learned number
per head if ``head_sink``) or "sigmoid" (every visible key weighs sigmoid(s + pb[n]), pb a number
per head if ``head_bias``; nothing is normalised over keys).  ``position``: a `PositionEncoding` whose
`rotary()` turns q and k (after their norm) by position - pairing, rotated size, scale and frequencies
are its own; ``out_bias``: whether the output projection has a bias (default: as ``bias``).  ``head_norm_weight``:
the norm per head multiplies by a learned weight of the head's size, one for q and one for k, shared by all heads.
``q_temp`` = (coef, every): q times 1 + coef ln(floor((position + 1) / every) + 1).  ``distance_table`` = (rows, far):
a learned table [rows, heads] of terms added to the scores by the bucket of the distance n = i - j - bucket(n) = n below
rows / 2, beyond that min(rows - 1, rows / 2 + floor(ln(n / (rows / 2)) / ln(far / (rows / 2)) * (rows - rows / 2))), made
once on the host in float64 for the distances 0 .. far.  ``element_gate``: the gate is a number per ELEMENT of the
concatenated heads (heads * v_head_dim logits of the mixer's input, further columns of the fused product) instead of
one per head.

Kernels: float32 and head sizes that are no multiples of 8 run on the plain kernel; bfloat16 on the
``mma.sync`` kernel of `ops.attention_window` (single-token steps share their keys out over CTAs),
except steps with prompt portions of head size 128 without gate and kept tokens, which take the
tcgen05 kernel (`ops.attention_tc`) with the same options; without a window it cuts a long key range
into slices (softmax weights only) so that the request's last tile does not set the kernel's time.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import ops
from .base import Mixer, PagedKVSpec, PositionEncoding, WeightSlot
from .linear import Linear


class GatedWindowAttention(Mixer):
    force_plain = False        # tests: bfloat16 through the plain kernel too, the twin of the tensor-core one
    tcgen05 = True             # tests: off, portions of head size 128 stay on the mma.sync kernel
    TC_SLICE = 512             # fewest keys a slice where a portion's key range is cut (softmax weights, no window)
    TC_SLICE_FILL = 148        # CTAs that the cut should reach: one an SM
    TC_MIN_ROWS = 64           # a step whose longest portion has more rows (tokens x heads of a group) takes the tcgen05 kernel
    graph_safe = True          # forward launches kernels over device tensors of the batch only

    def __init__(self, width: int, heads: int, kv_heads: int, head_dim: int, v_head_dim: int, dtype: torch.dtype, device,
                 prefix: str, scale: float, norm_eps: float, window: int = 0, keep_first: int = 0, own_kv: bool = True,
                 head_gate: bool = True, cache_window: Optional[int] = None, cache_keep_first: Optional[int] = None,
                 names=("q", "k", "v", "g", "o"), bias: bool = False, qk_norm: Optional[str] = "head", v_norm: bool = False,
                 softcap: float = 0.0, distance_bias: bool = False, weighting: str = "softmax", head_bias: bool = False,
                 extra_names=None, position: Optional[PositionEncoding] = None, head_sink: bool = False,
                 out_bias: Optional[bool] = None, head_norm_weight: bool = False, q_temp=None, distance_table=None,
                 element_gate: bool = False):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} kv heads")
        if max(head_dim, v_head_dim) > 256:
            raise ValueError(f"head sizes {head_dim} / {v_head_dim}: the attention kernels take sizes up to 256")
        self.width, self.heads, self.kv_heads, self.head_dim, self.v_head_dim = width, heads, kv_heads, head_dim, v_head_dim
        self.window, self.keep_first = int(window), int(keep_first) if window else 0
        # what the cache must hold: this layer's mask, widened by the layers that read its pages
        self.cache_window = self.window if cache_window is None else int(cache_window)
        self.cache_keep_first = self.keep_first if cache_keep_first is None else int(cache_keep_first)
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.own_kv, self.head_gate = own_kv, head_gate
        self.prefix, self.names, self.dtype = prefix, names, dtype
        self.q_cols = heads * head_dim
        self.kv_cols = kv_heads * (head_dim + v_head_dim) if own_kv else 0
        if element_gate and head_gate:
            raise ValueError("a gate per head or a gate per element, not both")
        self.element_gate = bool(element_gate)
        self.gate_cols = heads if head_gate else (heads * v_head_dim if element_gate else 0)
        self.proj = Linear(width, self.q_cols + self.kv_cols + self.gate_cols, dtype, device, bias=bias)
        self.out = Linear(heads * v_head_dim, width, dtype, device, bias=bias if out_bias is None else bool(out_bias))
        self.rotation = position.rotary() if position is not None else None
        if self.rotation is not None and self.rotation.dim > head_dim:
            raise ValueError(f"{self.rotation.dim} rotated dimensions exceed the head size {head_dim}")
        if bias and self.gate_cols and self.proj.bias.device.type != "meta":
            self.proj.bias[self.q_cols + self.kv_cols:].zero_()           # the gate logits have no bias
        if qk_norm not in (None, "head", "projection"):
            raise ValueError(f"qk_norm '{qk_norm}' is none of None, 'head', 'projection'")
        self.qk_norm, self.v_norm = qk_norm, bool(v_norm)
        f32 = dict(dtype=torch.float32, device=device)
        # the norm over a whole projection has a weight per column; the norm per head has none here
        self.q_norm_w = torch.empty((self.q_cols,), **f32) if qk_norm == "projection" else None
        self.k_norm_w = torch.empty((kv_heads * head_dim,), **f32) if qk_norm == "projection" and own_kv else None
        if head_norm_weight:
            if qk_norm != "head":
                raise ValueError("a weight of the head's size belongs to the norm per head")
            self.q_norm_w = torch.empty((head_dim,), **f32)
            self.k_norm_w = torch.empty((head_dim,), **f32) if own_kv else None
        self.q_temp = (float(q_temp[0]), int(q_temp[1])) if q_temp else None
        self.rel = self.rel_bucket = None
        if distance_table:
            rows, far = int(distance_table[0]), int(distance_table[1])
            half = rows // 2
            if rows < 2 or far <= half:
                raise ValueError(f"a table of {rows} distance terms up to distance {far}: it needs two rows at least and far beyond rows / 2")
            import math
            buckets = [n if n < half else min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))
                       for n in range(far + 1)]
            self.rel = torch.empty((rows, heads), **f32)
            self.rel_bucket = torch.tensor(buckets, dtype=torch.int32).to(device) if torch.device(device).type != "meta" else \
                torch.empty((far + 1,), dtype=torch.int32, device=device)
        self.r1 = torch.empty((heads,), **f32) if distance_bias else None
        self.r2 = torch.empty((heads,), **f32) if distance_bias else None
        self.pb = torch.empty((heads,), **f32) if head_bias else None
        if head_bias and weighting != "sigmoid":
            raise ValueError("a number per head added to the scores changes nothing under a softmax; it belongs to sigmoid weights")
        if head_sink and weighting != "softmax_sink":
            raise ValueError("a learned number per head for the denominator's extra term belongs to the weighting 'softmax_sink'")
        self.sink = torch.empty((heads,), **f32) if head_sink else None
        self.score = ops.ScoreOptions(softcap, self.r1, self.r2, self.pb, weighting, self.sink, self.rel, self.rel_bucket)
        self._scored = bool(softcap) or distance_bias or weighting != "softmax" or self.rel is not None
        # checkpoint names of what the options add, after the projections' own names
        self.extra_names = dict(bias=".b", q_norm=names[0] + ".norm", k_norm=names[1] + ".norm", r1="r1", r2="r2", head_bias="pb",
                                sink="sink", rel="rel")
        self.extra_names.update(extra_names or {})

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(self.kv_heads, self.head_dim, self.cache_window, self.cache_keep_first, self.v_head_dim)

    def weight_slots(self) -> List[WeightSlot]:
        p, (nq, nk, nv, ng, no) = self.prefix, self.names
        w = self.proj.weight
        slots = [WeightSlot(p + nq, w[:self.q_cols])]
        if self.own_kv:
            k_end = self.q_cols + self.kv_heads * self.head_dim
            slots += [WeightSlot(p + nk, w[self.q_cols:k_end]), WeightSlot(p + nv, w[k_end:self.q_cols + self.kv_cols])]
        if self.gate_cols:
            slots.append(WeightSlot(p + ng, w[self.q_cols + self.kv_cols:]))
        slots.append(WeightSlot(p + no, self.out.weight))
        x = self.extra_names
        if self.proj.bias is not None:
            b = self.proj.bias
            slots.append(WeightSlot(p + nq + x["bias"], b[:self.q_cols], "bias"))
            if self.own_kv:
                k_end = self.q_cols + self.kv_heads * self.head_dim
                slots += [WeightSlot(p + nk + x["bias"], b[self.q_cols:k_end], "bias"),
                          WeightSlot(p + nv + x["bias"], b[k_end:self.q_cols + self.kv_cols], "bias")]
        if self.out.bias is not None:
            slots.append(WeightSlot(p + no + x["bias"], self.out.bias, "bias"))
        if self.q_norm_w is not None:
            slots.append(WeightSlot(p + x["q_norm"], self.q_norm_w, "norm"))
        if self.k_norm_w is not None:
            slots.append(WeightSlot(p + x["k_norm"], self.k_norm_w, "norm"))
        if self.r1 is not None:
            slots += [WeightSlot(p + x["r1"], self.r1, "positive"), WeightSlot(p + x["r2"], self.r2, "positive")]
        if self.pb is not None:
            slots.append(WeightSlot(p + x["head_bias"], self.pb, "bias"))
        if self.sink is not None:
            slots.append(WeightSlot(p + x["sink"], self.sink, "bias"))
        if self.rel is not None:
            slots.append(WeightSlot(p + x["rel"], self.rel, "bias"))
        return slots

    def forward(self, x: torch.Tensor, batch, cache, residual: Optional[torch.Tensor] = None) -> Optional[ops.Partials]:
        if cache.writable != self.own_kv:
            raise ValueError("a mixer with key and value projections writes its cache layer; one without reads another's")
        T = x.shape[0]
        fused = self.proj.forward(x)
        q = torch.empty((T, self.q_cols), dtype=self.dtype, device=x.device)
        gate = torch.empty((T, self.heads), dtype=torch.float32, device=x.device) if self.head_gate else None
        table = batch.block_table(cache.group)
        ops.attn_prepare_ex(fused, self.q_norm_w, self.k_norm_w, self.qk_norm, self.norm_eps, batch.positions, batch.seq_of_token, table,
                            cache.page_size, cache.k, cache.v, q, gate, self.heads, self.kv_heads, self.head_dim, self.v_head_dim,
                            self.own_kv, v_norm=self.v_norm, rotation=self.rotation, q_temp=self.q_temp)
        score = self.score if self._scored else None
        a = torch.empty((T, self.heads * self.v_head_dim), dtype=self.dtype, device=x.device)
        G = self.heads // self.kv_heads
        if self.dtype == torch.bfloat16 and not self.force_plain and self.tcgen05 and self.head_dim == self.v_head_dim == 128 and \
                gate is None and self.keep_first == 0 and not batch.captured and batch.max_count * G > self.TC_MIN_ROWS and \
                ops.attention_tc_supported(128, cache.page_size):
            # prompt portions of head size 128: the tcgen05 kernel, rows in tiles of 256 per request
            tile_seq, tile_row0 = ops.row_tiles(batch, G, 256)
            # Few tiles far into a long context (a later portion of a long prompt) leave most SMs idle: softmax weights
            # without a window then take the key range in slices, as many as fill the chip, merged in ascending order.
            # A whole prompt has tiles enough and stays in one slice (cut at 512 keys, 2,048 tokens of 16 heads took 188
            # instead of 171 us: the slices' float32 outputs and their merge cost more than the even load gains).
            slices, slice_len = 1, 1 << 30
            fill = self.TC_SLICE_FILL // max(1, int(tile_seq.shape[0]) * self.kv_heads)
            if self.window == 0 and self.score.weighting != "sigmoid" and fill >= 2 and batch.max_kv_len > 2 * self.TC_SLICE and \
                    (self.score.weighting != "softmax_sink" or self.score.sink is not None):
                per = -(-batch.max_kv_len // min(32, fill))          # keys a slice if the chip is to be filled, in whole key tiles
                slice_len = max(self.TC_SLICE, (per + 127) // 128 * 128)
                slices = -(-batch.max_kv_len // slice_len)
            ops.attention_tc(q, cache.k, cache.v, a, tile_seq, tile_row0, batch.cu_seqlens, batch.kv_lens, table, cache.page_size, self.heads,
                             self.kv_heads, 128, self.window, self.scale, slices=slices,
                             slice_len=slice_len, rows_per_tile=256, score=score)
        elif self.dtype == torch.bfloat16 and not self.force_plain and \
                ops.attention_window_supported(self.head_dim, self.v_head_dim, self.heads, self.kv_heads):
            ops.attention_window(q, cache.k, cache.v, batch, table, cache.page_size, a, self.heads, self.kv_heads, self.head_dim,
                                 self.v_head_dim, self.window, self.keep_first, gate, self.scale, score)
        else:           # float32, and head sizes that are no multiple of 8
            ops.attention_plain_ex(q, cache.k, cache.v, batch.positions, batch.seq_of_token, table, cache.page_size, a, self.heads,
                                   self.kv_heads, self.head_dim, self.v_head_dim, self.window, self.keep_first, gate, self.scale, score)
        if self.element_gate:
            ops.gate_columns_mul(a, fused, self.q_cols + self.kv_cols)
        return self.out.forward(a, residual=residual)      # without bias and with many tokens the product adds itself to the stream
