"""Model parts (mixers, feed-forwards, norms, position encodings, blocks), their registries, and
the model assembled from a spec."""

from .base import (BLOCKS, DeferredSum, FEED_FORWARDS, INPUTS, MIXERS, NORMS, OUTPUTS, POSITION_ENCODINGS, Block, FeedForward,
                   InputPart, Mixer, Norm, OutputPart, Part, PositionEncoding, ResidualStream, StepContext, lookup,
                   register_block, register_feed_forward, register_input, register_mixer, register_norm,
                   register_output, register_position_encoding)
from . import norms, position, attention, latent, feed_forward, routed, recurrent, blocks, ends  # noqa: F401  (registers the built-in kinds)
from .attention import Attention
from .blocks import OutputNormResidual, PreNormResidual, SandwichResidual
from .ends import Embedding, NormHead
from .feed_forward import SwiGLU
from .latent import LatentAttention
from .routed import RoutedFeedForward
from .model import Model, cache_specs, expected_weights, run_order_for, tile_requests
from .norms import LayerNorm, RMSNorm
from .position import NoPosition, RopeNeox, RopePairs, rope_tables
from .recurrent import GatedLinearAttention, Mamba2, ParallelMixers

__all__ = [
    "Attention", "BLOCKS", "LatentAttention", "OutputNormResidual", "RoutedFeedForward", "DeferredSum", "GatedLinearAttention", "LayerNorm", "Mamba2", "ParallelMixers", "RopePairs",
    "SandwichResidual", "run_order_for", "Block", "Embedding", "FEED_FORWARDS", "FeedForward", "INPUTS", "InputPart", "MIXERS",
    "Mixer", "Model", "NORMS", "NoPosition", "Norm", "NormHead", "OUTPUTS", "OutputPart", "POSITION_ENCODINGS", "Part",
    "PositionEncoding", "PreNormResidual", "RMSNorm", "ResidualStream", "RopeNeox", "StepContext", "SwiGLU",
    "cache_specs", "expected_weights", "lookup", "register_block", "register_feed_forward", "register_input",
    "register_mixer", "register_norm", "register_output", "register_position_encoding",
    "rope_tables", "tile_requests",
]
