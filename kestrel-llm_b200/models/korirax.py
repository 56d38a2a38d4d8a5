"""The Korirax decoder assembled from parts.

The embedded tokens times a constant start the float32 stream.  Layers run in the order the configuration
lists them, a stretch of them several times over (same weights, a cache layer of its own for every run; in front
of every pass, the first too, a learned vector of that pass is added to every token of the stream); each is a
`ParallelBlock`: one RMSNorm, a mixer and a feed-forward that both read it and are added together, then a
per-layer token input (`TokenSideInput`).  A layer's mixer is one of

* ``attention``: `GatedWindowAttention` over all earlier tokens, without rotation: biased q, k, v projections, q and k
  normed per head with a learned weight of the head's size, a query temperature that grows with the position, a
  learned term per head and bucket of distances added to the scores, ordinary softmax, a gate per element of the
  concatenated heads;
* ``latent_attention``: `LatentAttention` with a rotated key part that all heads share beside the cached latent
  (interleaved rotary pairs, frequencies stretched by a ramp over the pair index), a gate per element;
* ``rglru``: `GatedDiagonalRecurrence`, decay rate 8.

Feed-forward: none, `GatedMLP` (SiLU), or `GroupRoutedExperts` (sigmoid router with a correction per expert and groups,
experts without a gate and with the exact gelu, one more expert that every token takes).  A final RMSNorm and the
output head.  Checkpoint tensors: ``embed``, ``loop.step``, ``side.embed``, ``l<i>.norm1``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``l<i>.side.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import torch

from ..config.korirax_config import NAME, BiasedAttentionSpec, DenseSpec, KoriraxConfig, MoeSpec, RglruSpec, RotaryLatentSpec
from ..config.registry import register_architecture
from ..parts import (GatedDiagonalRecurrence, GatedMLP, GatedWindowAttention, GroupRoutedExperts, LatentAttention, LMHead, ParallelBlock,
                     RampScaling, RMSNorm, RotaryInterleaved, StreamRows, TokenEmbedding, TokenSideInput, TokenTable)
from .decoder import DecoderModel, LayerCall

DECAY_RATE = 8.0        # the recurrence's decay is exp(-DECAY_RATE * r * softplus(lam))


def build_korirax(config: KoriraxConfig, dtype: torch.dtype, device) -> DecoderModel:
    c = config
    W, eps, L = c.hidden_size, c.norm_eps, len(c.layers)
    emb = TokenEmbedding(c.vocab_size, W, dtype, device, "embed", scale=c.embedding_scale)
    table = TokenTable(c.vocab_size, L * c.side_dim, dtype, device, "side.embed") if c.side_dim else None
    blocks = []
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer.mixer
        if isinstance(m, BiasedAttentionSpec):
            if not m.bias_rows:
                raise ValueError(f"layer {i}: the rows of the table of distance terms are unknown (KoriraxConfig.with_tensor_shapes)")
            mixer = GatedWindowAttention(W, m.heads, m.kv_heads, m.dim, m.vdim, dtype, device, p + "mix.", m.scale, eps, window=0,
                                         head_gate=False, element_gate=True, bias=True, out_bias=False, qk_norm="head",
                                         head_norm_weight=True, q_temp=m.q_temp, distance_table=(m.bias_rows, m.bias_max))
        elif isinstance(m, RotaryLatentSpec):
            position = None
            if m.rot is not None and m.rot_dim:
                s = m.rot.scaling
                ramp = RampScaling(s.factor, s.original, s.fast, s.slow, m.rot.dims, m.rot.base) if s is not None else None
                position = RotaryInterleaved(m.rot_dim, m.rot.base, device, rotary_dim=m.rot.dims, scaling=ramp,
                                             scale=ramp.magnitude if ramp is not None else 1.0)
            mixer = LatentAttention(W, m.heads, m.dim, m.vdim, m.q_rank, m.kv_rank, dtype, device, p + "mix.", m.scale, eps, window=0,
                                    head_gate=False, element_gate=True, rot_dim=m.rot_dim, position=position)
        else:
            assert isinstance(m, RglruSpec)
            mixer = GatedDiagonalRecurrence(W, m.width, m.blocks, m.taps, dtype, device, p + "mix.", rate=DECAY_RATE)
        f = layer.mlp
        if f is None:
            ffn = None
        elif isinstance(f, DenseSpec):
            ffn = GatedMLP(W, f.ff, dtype, device, p + "mlp.", names=("gate", "up", "down"))
        else:
            assert isinstance(f, MoeSpec)
            ffn = GroupRoutedExperts(W, f.ff, f.experts, f.top, dtype, device, p + "mlp.", groups=f.groups, keep=f.keep, scale=f.scale,
                                     activation="gelu", shared_inner=f.shared_ff)
        side = TokenSideInput(W, c.side_dim, table, i * c.side_dim, eps, dtype, device, p + "side.") if table is not None else None
        blocks.append(ParallelBlock(RMSNorm(W, eps, device, p + "norm1"), mixer, ffn, side, dtype))
    # every run of a layer has a cache layer of its own; a pass of the loop opens with its learned vector
    order = [LayerCall(block=i, cache=n, add_row=-1 if t is None else t) for n, (i, t) in enumerate(c.layer_runs())]
    rows = StreamRows(c.loop_passes, W, device, "loop.step") if c.loop_passes else None
    return DecoderModel(c, dtype, device, emb, None, blocks, order, RMSNorm(W, eps, device, "final.norm"),
                        LMHead(c.vocab_size, W, dtype, device, "head"), shared_parts=[table] if table is not None else [],
                        stream_rows=rows, optional_tensors=[] if rows is not None else ["loop.step"])


register_architecture(NAME, KoriraxConfig, build_korirax)
