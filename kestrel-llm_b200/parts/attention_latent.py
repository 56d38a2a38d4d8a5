"""Softmax attention whose keys and values of all heads are expanded from one latent vector a
token, and only that vector is cached.

With h the mixer's input, H heads, d query/key dimensions and dv value dimensions a head:

    cq = rmsnorm(W_dq h) * w_q                  query latent, q_rank numbers
    q  = W_uq cq                                [H, d]
    c  = rmsnorm(W_dkv h) * w_kv                key/value latent, kv_rank numbers - what the cache keeps
    k_n = Uk_n c,  v_n = Uv_n c                 head n's rows of W_uk [H d, kv_rank] and W_uv [H dv, kv_rank]
    p   = softmax_j(q_n . k_nj * scale)         over the window: query i sees key j if 0 <= i - j < window (0: all)
    y   = W_o concat_n( sigmoid(W_g h)_n * sum_j p_j v_nj )

Heads are not rotated unless the mixer is built with ``rot_dim`` > 0: a head's query then has ``rot_dim`` more dimensions behind
its ``d`` unrotated ones, W_dkv has ``rot_dim`` more rows behind the latent's - one key part that ALL heads share, not normed -,
both are turned by position as ``position`` (a `PositionEncoding` with a `rotary()`) says, and the score is
(q_n[:d] . k_nj + q_n[d:] . kr_j) * scale.  The cache row of a token is then [c | kr], and the query that meets it
[Uk_n^T q_n[:d] | q_n[d:]]: attention still runs over the cache rows themselves, as one key/value head whose keys are the rows
of kv_rank + rot_dim numbers and whose values are the rows' first kv_rank (the kernels take the V plane's row length apart from
the value size).  ``element_gate``: the gate is a
number per element of the concatenated heads instead of one per head.

Since q_n . k_nj = (Uk_n^T q_n) . c_j and sum_j p_j v_nj = Uv_n sum_j p_j c_j,
attention runs over the cached latents themselves as ONE key/value head of size kv_rank shared by
all query heads (`PagedKVSpec.values_are_keys`): the queries are taken into the latent space by a
head-wise product before it, the mixed latents out of it by another one afterwards.  W_dq, W_dkv
and W_g are one fused product.  The gate may be absent (``head_gate=False``).

One exception, for speed: a bfloat16 step in which every request STARTS (no request has tokens in
the cache yet) and brings a long portion, with d = dv = 128.  All the keys its queries can see are
then the step's own, so they are expanded once - k and v of the step's tokens from one fused product
of their latents, into pages of a scratch cache - and the tcgen05 attention kernel runs over them
with H key heads of 128 instead of one of ``kv_rank``; the gate follows as a kernel of its own.  The
latents still go to the real cache, from which every later step reads.  The two forms differ by
rounding only.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import ops
from .base import Mixer, PagedKVSpec, WeightSlot
from .linear import Linear


class LatentAttention(Mixer):
    force_plain = False        # tests: bfloat16 through the plain attention kernel too
    expand_prompts = True      # tests: off, starting portions too run over the cached latents
    EXPAND_MIN_TOKENS = 64     # a step whose longest portion has more tokens may take the expanded form
    graph_safe = True          # forward launches kernels over device tensors of the batch only (the expanded form reads the
                               # host's copy of the step, and is never taken while a step is recorded)

    def __init__(self, width: int, heads: int, head_dim: int, v_head_dim: int, q_rank: int, kv_rank: int, dtype: torch.dtype, device,
                 prefix: str, scale: float, norm_eps: float, window: int = 0, head_gate: bool = True,
                 names=("dq", "uq", "dkv", "uk", "uv", "g", "o"), rot_dim: int = 0, position=None, element_gate: bool = False):
        if kv_rank + rot_dim > 576:
            raise ValueError(f"a cached row of {kv_rank} + {rot_dim} numbers: the plain attention kernel takes head sizes up to 576 "
                             f"(the tensor-core kernels up to 256)")
        if element_gate and head_gate:
            raise ValueError("a gate per head or a gate per element, not both")
        self.rot_dim, self.element_gate = int(rot_dim), bool(element_gate)
        self.rotation = position.rotary() if position is not None and rot_dim else None
        if self.rotation is not None and self.rotation.dim > rot_dim:
            raise ValueError(f"{self.rotation.dim} rotated dimensions exceed the rotated part of {rot_dim}")
        self.row = kv_rank + self.rot_dim                      # what the cache keeps of a token
        self.width, self.heads, self.head_dim, self.v_head_dim = width, heads, head_dim, v_head_dim
        self.q_rank, self.kv_rank, self.window = q_rank, kv_rank, int(window)
        self.scale, self.norm_eps, self.head_gate = float(scale), float(norm_eps), head_gate
        self.prefix, self.names, self.dtype = prefix, names, dtype
        self.gate_cols = heads if head_gate else (heads * v_head_dim if element_gate else 0)
        self.down = Linear(width, q_rank + self.row + self.gate_cols, dtype, device)
        self.up_q = Linear(q_rank, heads * (head_dim + self.rot_dim), dtype, device)
        self.up_kv = Linear(kv_rank, heads * (head_dim + v_head_dim), dtype, device)     # rows [k | v]: one product where both are expanded
        self.up_k_w = self.up_kv.weight[:heads * head_dim]                  # used transposed, head by head
        self.up_v_w = self.up_kv.weight[heads * head_dim:]
        self.out = Linear(heads * v_head_dim, width, dtype, device)
        self.q_norm_w = torch.empty((q_rank,), dtype=torch.float32, device=device)
        self.kv_norm_w = torch.empty((kv_rank,), dtype=torch.float32, device=device)

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(1, self.row, self.window, 0, self.row, values_are_keys=True)

    def weight_slots(self) -> List[WeightSlot]:
        p, (dq, uq, dkv, uk, uv, g, o) = self.prefix, self.names
        w, r = self.down.weight, self.q_rank + self.row
        slots = [WeightSlot(p + dq, w[:self.q_rank]), WeightSlot(p + dkv, w[self.q_rank:r]),
                 WeightSlot(p + dq + ".norm", self.q_norm_w, "norm"), WeightSlot(p + dkv + ".norm", self.kv_norm_w, "norm"),
                 WeightSlot(p + uq, self.up_q.weight), WeightSlot(p + uk, self.up_k_w), WeightSlot(p + uv, self.up_v_w),
                 WeightSlot(p + o, self.out.weight)]
        if self.gate_cols:
            slots.append(WeightSlot(p + g, w[r:]))
        return slots

    def forward(self, x: torch.Tensor, batch, cache, residual: Optional[torch.Tensor] = None) -> Optional[ops.Partials]:
        T, H, R = x.shape[0], self.heads, self.kv_rank
        fused = self.down.forward(x)
        cq = torch.empty((T, self.q_rank), dtype=self.dtype, device=x.device)
        gate = torch.empty((T, H), dtype=torch.float32, device=x.device) if self.head_gate else None
        table = batch.block_table(cache.group)
        expand = (self.dtype == torch.bfloat16 and not self.force_plain and self.expand_prompts and self.head_dim == self.v_head_dim == 128
                  and self.rot_dim == 0 and not self.element_gate and not batch.captured and batch.max_count > self.EXPAND_MIN_TOKENS and all(s == 0 for s in batch.starts)
                  and ops.attention_tc_supported(128, cache.page_size))
        c_rows = torch.empty((T, R), dtype=self.dtype, device=x.device) if expand else None
        ops.latent_prepare(fused, self.q_norm_w, self.kv_norm_w, self.norm_eps, batch.positions, batch.seq_of_token, table, cache.page_size,
                           cache.k, cq, gate, kv_out=c_rows, rot_cols=self.rot_dim, rotation=self.rotation)
        q = self.up_q.forward(cq).reduce(self.dtype)                           # [T, H (d + rot_dim)]
        if expand:
            return self._forward_expanded(q, c_rows, gate, batch, cache.page_size, residual)
        D, d = self.row, self.head_dim
        if self.rot_dim:
            # a head's query in the space of the cache rows: [Uk_n^T q_n[:d] | q_n[d:] turned by position]
            q_lat = torch.empty((T, H * D), dtype=self.dtype, device=x.device)
            ops.head_gemm(q, self.up_k_w, H, w_kn=True, out=q_lat, x_head_stride=d + self.rot_dim, out_head_stride=D)
            ops.latent_rotate_queries(q, H, d, self.rot_dim, q_lat, R, batch.positions, self.rotation)
        else:
            q_lat = ops.head_gemm(q, self.up_k_w, H, w_kn=True)                # [T, H kv_rank]: Uk_n^T q_n
        # keys are whole cache rows, values their first kv_rank numbers: the V plane is the K plane with rows of D numbers
        a = torch.empty((T, H * R), dtype=self.dtype, device=x.device)
        if self.dtype == torch.bfloat16 and not self.force_plain and ops.attention_window_supported(D, R, H, 1):
            ops.attention_window(q_lat, cache.k, cache.k, batch, table, cache.page_size, a, H, 1, D, R, self.window, 0, gate, self.scale,
                                 v_ld=D)
        else:
            ops.attention_plain_ex(q_lat, cache.k, cache.k, batch.positions, batch.seq_of_token, table, cache.page_size, a, H, 1, D, R,
                                   self.window, 0, gate, self.scale, v_ld=D)
        o = ops.head_gemm(a, self.up_v_w, H, w_kn=False)                       # [T, H dv]: Uv_n (mixed latent)
        if self.element_gate:
            ops.gate_columns_mul(o, fused, self.q_rank + self.row)
        return self.out.forward(o, residual=residual)      # many tokens: the product adds itself to the stream

    def _forward_expanded(self, q, c_rows, gate, batch, page: int, residual):
        """Starting portions: keys and values of the step's tokens expanded into scratch pages, tcgen05 attention over them."""
        T, H, dev = q.shape[0], self.heads, q.device
        kept = batch.__dict__.setdefault("_scratch_tables", {})
        if page not in kept:         # every request's tokens from a page border, in the order of the step
            blocks = [(n + page - 1) // page for n in batch.counts]
            rows = torch.zeros((len(blocks), max(blocks)), dtype=torch.int32)
            at = 0
            for i, b in enumerate(blocks):
                rows[i, :b] = torch.arange(at, at + b, dtype=torch.int32)
                at += b
            kept[page] = (rows.to(dev, non_blocking=True), at)
        scratch_table, n_pages = kept[page]
        k_pages = torch.empty((n_pages, H, page, 128), dtype=self.dtype, device=dev)
        v_pages = torch.empty((n_pages, H, page, 128), dtype=self.dtype, device=dev)
        kv = self.up_kv.forward(c_rows)                                        # columns [k: H d | v: H dv]
        no_q = torch.empty((T, 0), dtype=self.dtype, device=dev)
        ops.attn_prepare_ex(kv, None, None, None, self.norm_eps, batch.positions, batch.seq_of_token, scratch_table, page, k_pages, v_pages,
                            no_q, None, 0, H, 128, 128, True)
        a = torch.empty((T, H * 128), dtype=self.dtype, device=dev)
        tile_seq, tile_row0 = ops.row_tiles(batch, 1, 256)
        ops.attention_tc(q, k_pages, v_pages, a, tile_seq, tile_row0, batch.cu_seqlens, batch.kv_lens, scratch_table, page, H, H, 128,
                         self.window, self.scale, rows_per_tile=256)
        if gate is not None:
            ops.head_scale(a, gate, H)
        return self.out.forward(a, residual=residual)
