from .base import (Block, CacheSpec, CombinedSpec, FeedForward, FixedStateSpec, Mixer, Norm, PagedKVSpec, Part,
                   PositionEncoding, Rotation, WeightSlot)
from .linear import Linear
from .norm import RMSNorm
from .rotary import FrequencyScaling, RampScaling, NoPositionEncoding, RotaryHalf, RotaryInterleaved, SinusoidalPositions
from .attention import GroupedQueryAttention
from .mlp import DenseMLP, GatedMLP
from .attention_gated import GatedWindowAttention
from .attention_latent import LatentAttention
from .delta import ChannelDeltaMixer
from .recurrence import ForgetGateRecurrence, RemovalDeltaMixer
from .parallel import ParallelMixers
from .moe import GroupRoutedExperts, RoutedExperts
from .rglru import GatedDiagonalRecurrence
from .side_input import TokenSideInput, TokenTable
from .block import ParallelBlock, PreNormBlock, SandwichBlock
from .embedding import LMHead, StreamRows, TokenEmbedding

__all__ = ["Block", "CacheSpec", "FeedForward", "FixedStateSpec", "Mixer", "Norm", "PagedKVSpec", "Part",
           "PositionEncoding", "Rotation", "WeightSlot", "Linear", "RMSNorm", "NoPositionEncoding", "RotaryHalf", "RotaryInterleaved",
           "GroupedQueryAttention", "GatedMLP", "PreNormBlock", "LMHead", "TokenEmbedding", "SinusoidalPositions",
           "GatedWindowAttention", "LatentAttention", "ChannelDeltaMixer", "RoutedExperts", "TokenSideInput", "TokenTable", "ParallelBlock",
           "CombinedSpec", "FrequencyScaling", "DenseMLP", "ForgetGateRecurrence", "RemovalDeltaMixer", "ParallelMixers", "SandwichBlock",
           "RampScaling", "GroupRoutedExperts", "GatedDiagonalRecurrence", "StreamRows"]
