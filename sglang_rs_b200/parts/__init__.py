from .attention import AttentionNames, GroupedQueryAttention
from .base import (CacheNeed, FeedForward, Mixer, Norm, NormedDelta, PagedKV, Part, PositionEncoding, RequestState,
                   TensorSpec, matrix_to, scale_to)
from .block import ParallelBlock, PreNormBlock, SandwichBlock
from .latent_attention import LatentAttention, LatentAttentionNames
from .loop import PassEntry, PassSum
from .moe import RoutedExperts
from .embedding import OutputHead, PairTokenEmbedding, TokenEmbedding
from .hyper import StreamBlock, StreamConnection, StreamNames, StreamSumNorm, StreamUpdate
from .lightning import LightningAttention, LightningNames
from .mlp import GatedMlp, GatedMlpNames, PlainMlp
from .mamba import MambaMixer, MambaNames
from .norm import GroupedRmsNorm, LayerNorm, RmsNorm
from .side import TokenSideInput, TokenSideNames
from .rope import NoPositionEncoding, RotaryEncoding, WavelengthScaling

__all__ = [
    "AttentionNames", "GroupedQueryAttention", "CacheNeed", "FeedForward", "Mixer", "Norm", "PagedKV", "Part",
    "PositionEncoding", "RequestState", "TensorSpec", "matrix_to", "scale_to", "PreNormBlock", "OutputHead",
    "TokenEmbedding", "GatedMlp", "GatedMlpNames", "RmsNorm", "NoPositionEncoding", "RotaryEncoding", "NormedDelta",
    "SandwichBlock", "LatentAttention", "LatentAttentionNames", "PassEntry", "PassSum", "RoutedExperts", "LayerNorm",
    "PairTokenEmbedding", "StreamBlock", "StreamConnection", "StreamNames", "StreamSumNorm", "StreamUpdate",
    "LightningAttention", "LightningNames", "PlainMlp", "WavelengthScaling",
    "ParallelBlock", "GroupedRmsNorm", "MambaMixer", "MambaNames", "TokenSideInput", "TokenSideNames",
]
