from .attention import Attention, paged_attention
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Delta, FeedForward, Mixer,
                   PagedKVSpec, Part, Registry, StateSpec)
from .block import Block, NormAfterBlock, ParallelBlock, PostNormBlock, PreNormBlock, ReentryBlock, ResidualStream
from .conv import InputConv
from .delta_rule import GatedDeltaRule
from .diff_attention import DifferentialAttention
from .embedding import Embedding, OutputHead
from .ffn import ClampedGatedFFN, DenseFFN, GatedFFN
from .grouped_attention import GroupedAttention
from .hgrn2 import HGRN2
from .latent_attention import LatentAttention
from .moe import RoutedExperts
from .norm import LayerNorm, NoNorm, Norm, OffsetRMSNorm, RMSNorm, ScalarRMSNorm
from .side_by_side import SideBySide
from .position import LearnedPositions, NoPositions, PositionEncoding, RotaryHalves, RotaryPairs

__all__ = ["Attention", "BLOCKS", "Block", "Delta", "DenseFFN", "Embedding", "FEED_FORWARDS", "FeedForward",
           "LayerNorm", "LearnedPositions", "MIXERS", "Mixer", "NORMS", "NoNorm", "NoPositions", "Norm",
           "OutputHead", "POSITION_ENCODINGS", "PagedKVSpec", "Part", "PositionEncoding", "PostNormBlock",
           "PreNormBlock", "RMSNorm", "Registry", "ResidualStream", "StateSpec", "paged_attention",
           "DifferentialAttention", "GatedFFN", "HGRN2", "InputConv", "NormAfterBlock", "RotaryPairs", "ScalarRMSNorm",
           "LatentAttention", "OffsetRMSNorm", "ClampedGatedFFN", "GatedDeltaRule", "GroupedAttention", "SideBySide", "ParallelBlock", "ReentryBlock", "RotaryHalves", "RoutedExperts"]
