"""The Toredra decoder assembled from parts.

The embedded tokens start the float32 stream (no position vector: the attention rotates its
heads).  Layers run in the order the configuration lists them, a stretch of them several times
over (same weights, a cache layer of its own for every run; the embedded tokens are added to the
stream again in front of every further pass); each is a `SandwichBlock`: a norm in front of a
sublayer, the sublayer's result gated by sigmoid(W h + b) of its own input h, normed again, then
added.  A layer's mixer is one of

* ``parallel``: `ParallelMixers` - a `GatedWindowAttention` over all earlier tokens (biased q, k, v
  projections, interleaved rotary pairs on the first dimensions of a head with stretched long
  wavelengths, a softmax whose denominator has a learned term per head) beside a
  `ForgetGateRecurrence`, each normed, then averaged;
* ``general_delta``: `RemovalDeltaMixer`, decay rate exp(-1/2).

Feed-forward: `DenseMLP` with the square of relu.  A final RMSNorm; the output head is the
embedding table, its logits scaled and then capped by a tanh.  Checkpoint tensors: ``embed``,
``l<i>.norm1``, ``norm1b``, ``norm2``, ``norm2b``, ``rg1``, ``rg1.b``, ``rg2``, ``rg2.b``, ``l<i>.mix.*``,
``l<i>.mlp.{up,down}``, ``final.norm``.
"""
from __future__ import annotations

import math

import torch

from ..config.registry import register_architecture
from ..config.toredra_config import NAME, GeneralDeltaSpec, ParallelSpec, ToredraConfig
from ..parts import (DenseMLP, ForgetGateRecurrence, FrequencyScaling, GatedWindowAttention, Linear, LMHead, ParallelMixers,
                     RemovalDeltaMixer, RMSNorm, RotaryInterleaved, SandwichBlock, TokenEmbedding)
from .decoder import DecoderModel, LayerCall

DECAY_RATE = math.exp(-0.5)       # the delta rule's decay is exp(-DECAY_RATE * sigmoid(.)) per token and key channel


def build_toredra(config: ToredraConfig, dtype: torch.dtype, device) -> DecoderModel:
    c = config
    W, eps = c.hidden_size, c.norm_eps
    blocks, optional = [], []
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer.mixer
        if isinstance(m, ParallelSpec):
            a, b = m.left, m.right
            position = None
            if a.rot is not None:
                scaling = FrequencyScaling(*a.rot.scaling) if a.rot.scaling is not None else None
                position = RotaryInterleaved(a.dim, a.rot.base, device, rotary_dim=a.rot.dims, scaling=scaling)
            left = GatedWindowAttention(W, a.heads, a.kv_heads, a.dim, a.vdim, dtype, device, p + "mix.left.", a.scale, eps, window=0,
                                        head_gate=False, bias=True, out_bias=False, qk_norm=None, weighting="softmax_sink", head_sink=True,
                                        position=position)
            right = ForgetGateRecurrence(W, b.heads, b.dim, b.vdim, eps, dtype, device, p + "mix.right.")
            mixer = ParallelMixers(left, right, W, eps, device, p + "mix.")
        else:
            assert isinstance(m, GeneralDeltaSpec)
            if not m.decay_rank:
                raise ValueError(f"layer {i}: the rank of the decay's projection is unknown (ToredraConfig.with_tensor_shapes)")
            mixer = RemovalDeltaMixer(W, m.heads, m.dim, m.decay_rank, DECAY_RATE, eps, dtype, device, p + "mix.")
        ffn = norm2 = norm2b = gate2 = None
        if layer.mlp is not None:
            ffn = DenseMLP(W, layer.mlp.ff, dtype, device, p + "mlp.", activation="relu2")
            norm2, norm2b = RMSNorm(W, eps, device, p + "norm2"), RMSNorm(W, eps, device, p + "norm2b")
            gate2 = Linear(W, W, dtype, device, bias=True)
        else:
            optional += [p + "norm2", p + "norm2b", p + "rg2", p + "rg2.b"]      # a layer without feed-forward has no use for them
        blocks.append(SandwichBlock(RMSNorm(W, eps, device, p + "norm1"), mixer, RMSNorm(W, eps, device, p + "norm1b"),
                                    Linear(W, W, dtype, device, bias=True), norm2, ffn, norm2b, gate2, dtype, p))
    # every run of a layer has a cache layer of its own; a further pass starts with the embedded tokens added in again
    order = [LayerCall(block=i, cache=n, add_embedding=again) for n, (i, _rep, again) in enumerate(c.layer_runs())]
    emb = TokenEmbedding(c.vocab_size, W, dtype, device, "embed")
    return DecoderModel(c, dtype, device, emb, None, blocks, order, RMSNorm(W, eps, device, "final.norm"),
                        LMHead(c.vocab_size, W, dtype, device, "head", tied_to=emb, scale=c.logit_scale, softcap=c.logit_softcap),
                        optional_tensors=optional)


register_architecture(NAME, ToredraConfig, build_toredra)
