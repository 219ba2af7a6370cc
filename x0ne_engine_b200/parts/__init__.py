"""The parts layers are made of, and their registries."""
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, OPENERS, PART_REGISTRIES, POSITIONS, Block, BuildEnv,
                   CacheNeed, Embedding, FeedForward, Head, Mixer, Norm, Opener, Part, PositionEncoding, Registry)
from .linear import Linear
from . import attention, block, diff_attention, distance_attention, embedding, latent_attention, masked_attention, mlp, moe, norm, recurrent, rope, selective_scan, window_attention  # noqa: F401  (registers the built-in parts)
from .attention import GQAttention
from .block import ParallelBlock, PreNormBlock, PreNormMixerBlock, SandwichBlock
from .latent_attention import LatentAttention
from .masked_attention import MaskedAttention
from .distance_attention import DistanceBiasAttention
from .diff_attention import DifferentialAttention
from .selective_scan import SelectiveScan
from .embedding import LMHead, PassOpener, TokenEmbedding
from .mlp import BiasedMLP, ClippedGLU, SwiGLU
from .recurrent import MatrixStateRecurrence
from .moe import RoutedExperts
from .norm import PostNormed, RMSNorm
from .window_attention import SinkWindowAttention
from .rope import NoPosition, Rope, YarnRope, inv_freq_f32, yarn_frequencies

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "PART_REGISTRIES", "POSITIONS", "Block",
           "BuildEnv", "CacheNeed", "Embedding", "FeedForward", "Head", "Mixer", "Norm", "Part", "PositionEncoding",
           "Registry", "Linear", "GQAttention", "OPENERS", "Opener", "PassOpener", "DistanceBiasAttention", "BiasedMLP",
           "MatrixStateRecurrence", "PreNormMixerBlock", "DifferentialAttention", "SelectiveScan",
           "PreNormBlock", "ParallelBlock", "SandwichBlock", "SinkWindowAttention", "RoutedExperts", "PostNormed", "MaskedAttention", "LatentAttention", "ClippedGLU", "YarnRope", "yarn_frequencies", "LMHead", "TokenEmbedding", "SwiGLU", "RMSNorm", "NoPosition", "Rope", "inv_freq_f32"]
