"""Parts a model is put together from: norm, position encoding, mixer, feed-forward,
their arrangement in a block, embedding and output head."""
from .base import (BuildContext, FeedForward, KVSpec, LayerBinding, Mixer, Norm, Part, PositionEncoding,
                   StateSpec, WeightSpec)
from .stream import ResidualStream
from .norms import RMSNormGrouped, RMSNormL2, RMSNormMeanEps, RMSNormOnePlus, RMSNormScalar
from .positions import RotaryHalf, RotaryInterleaved, RotaryRescaled
from .attention import GqaAttention
from .feed_forward import ActMLP, ClampedGLU, RoutedExperts, SwiGLU
from .short_conv import CausalConv
from .window_attention import BiasedWindowAttention, ValueShare
from .delta_rule import ChannelDeltaRule, HeadDecayDeltaRule
from .linear_attention import DecayLinearAttention
from .latent_attention import LatentAttention
from .diff_attention import DifferentialAttention
from .gated_recurrence import ForgetGateRecurrence
from .gated_linear_attention import GatedLinearAttention
from .sink_attention import TiedValueAttention
from .state_space import SelectiveStateSpace
from .side_by_side import SideBySide
from .block import Block
from .embedding import Embedding, LMHead, PairHashEmbedding

__all__ = ["BuildContext", "FeedForward", "KVSpec", "LayerBinding", "Mixer", "Norm", "Part",
           "PositionEncoding", "StateSpec", "WeightSpec", "ResidualStream", "RMSNormL2", "RMSNormMeanEps", "RMSNormOnePlus", "ClampedGLU", "CausalConv",
           "BiasedWindowAttention", "ValueShare", "ChannelDeltaRule", "HeadDecayDeltaRule", "DecayLinearAttention", "LatentAttention", "RoutedExperts",
           "RotaryRescaled", "RotaryHalf",
           "RotaryInterleaved", "GqaAttention", "SwiGLU", "Block", "Embedding", "LMHead", "RMSNormScalar", "ActMLP",
           "DifferentialAttention", "ForgetGateRecurrence", "GatedLinearAttention", "TiedValueAttention", "SelectiveStateSpace",
           "SideBySide", "PairHashEmbedding", "RMSNormGrouped"]
