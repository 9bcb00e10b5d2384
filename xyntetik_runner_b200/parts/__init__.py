"""Parts that layers are put together from; importing this package registers the built-in kinds."""
from .base import (Block, FeedForward, KVNeed, Mixer, Norm, Part, PositionEncoding, Rotary, Runtime, StateNeed, kinds, make,
                   register_block, register_feed_forward, register_mixer, register_norm, register_position)
from .attention import GQAAttention
from .block import OutputNormBlock, ParallelBlock, PreNormBlock
from .decay_attention import DecayLinearAttention
from .delta import GatedDelta
from .embedding import Embedding, Head, PairEmbedding
from .feed_forward import GatedFeedForward, MLP, SwiGLU
from .latent_attention import LatentAttention
from .linear import Linear
from .mlstm import MLSTM
from .moe import RoutedExperts
from .norm import RMSNorm, ScalarRMSNorm
from .position import NoPosition, Rope, YarnRope
from .rglru import GatedLinearRecurrence
from .side_by_side import SideBySide
from .stream import DepthAverage, StreamJoin, StreamStep
