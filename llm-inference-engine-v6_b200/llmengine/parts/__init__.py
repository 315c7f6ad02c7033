"""Parts a layer is put together from: mixers, feed-forwards, norms, position encodings, blocks."""
from . import (attention, block, embedding, gated_attention, latent_attention, linear_state, mixer_pair, mlp, norm, position, routed_mlp,
               selective_scan, token_side)  # noqa: F401  (registers the built-in parts)
from .base import (Block, BuildEnv, Embedding, FeedForward, Head, KVNeed, LayerCache, Mixer, Norm, NormalizedRows,
                   Part, PositionEncoding, Residual, StateNeed, TokenInput)
from .registry import build_part, part_class, register_part
from .spec import (AttentionSpec, BlockSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec, LatentAttentionSpec, LayerRun, ModelSpec,
                   NormSpec, PositionSpec, RoutedMLPSpec, ScaledRotarySpec, TensorNeed, TokenSideSpec)

__all__ = ["Block", "BuildEnv", "Embedding", "FeedForward", "Head", "KVNeed", "LayerCache", "Mixer", "Norm", "NormalizedRows", "Part", "PositionEncoding",
           "Residual", "StateNeed", "build_part", "part_class", "register_part", "AttentionSpec", "BlockSpec",
           "EmbeddingSpec", "GatedMLPSpec", "HeadSpec", "LayerRun", "ModelSpec", "NormSpec", "PositionSpec",
           "TensorNeed", "TokenInput", "LatentAttentionSpec", "RoutedMLPSpec", "ScaledRotarySpec", "TokenSideSpec"]
