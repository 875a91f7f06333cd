"""Parts a model is put together from; importing this package registers the built-in ones."""

from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheSpec,
                   Embedding, FeedForward, Head, IntoNorm, LayerBinding, Mixer, Norm, Part, PositionEncoding, Registry, Runtime,
                   StateSpec, WeightSpec)
from .attention import PagedAttention
from .block import BranchNormBlock, ParallelBlock, PreNormBlock
from .embedding import LMHead, SummedEmbedding, TokenEmbedding
from .mlp import ActivatedFeedForward, GatedFeedForward, SwiGLUFeedForward
from .experts import RoutedExperts
from .norm import GroupRMSNorm, RMSNorm, StreamRounding
from .state_space import StateSpaceMixer
from .recurrent import (ConvolvedInput, DecayedLinearAttention, GatedLinearRecurrenceMixer, GatedRecurrenceMixer,
                        MatrixMemoryMixer, ParallelMixers)
from .latent_attention import LatentAttention
from .rotary import NoPositionEncoding, RotaryEncoding, YarnRotaryEncoding
from .streams import ConnectedNorm, HyperConnectionBlock, StreamWrite

__all__ = ["BLOCKS", "EMBEDDINGS", "HEADS", "Embedding", "Head", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "CacheSpec",
           "FeedForward", "IntoNorm", "LayerBinding", "Mixer", "Norm", "Part", "PositionEncoding", "Registry",
           "Runtime", "StateSpec", "WeightSpec", "PagedAttention", "PreNormBlock", "LMHead",
           "TokenEmbedding", "SwiGLUFeedForward", "GatedFeedForward", "RMSNorm", "NoPositionEncoding", "RotaryEncoding", "YarnRotaryEncoding", "ConnectedNorm",
           "HyperConnectionBlock", "StreamWrite", "BranchNormBlock", "GroupRMSNorm", "StreamRounding", "RoutedExperts",
           "StateSpaceMixer", "SummedEmbedding", "ActivatedFeedForward", "ConvolvedInput", "GatedRecurrenceMixer",
           "MatrixMemoryMixer", "LatentAttention", "ParallelBlock", "DecayedLinearAttention", "GatedLinearRecurrenceMixer",
           "ParallelMixers"]
