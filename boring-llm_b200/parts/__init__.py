from .base import Part, StepContext, StepPlan, to_device_matrix, to_device_vector
from .linear import linear
from .norm import RMSNorm, LayerNorm
from .rotary import RotaryTable
from .attention import Mixer, GQAAttention, GatedSinkAttention, ChunkedTalkingAttention, ParallelMixers
from .recurrent import (GatedLinearAttention, ChannelDeltaRule, MatrixMemory, ShiftedDecayRecurrence, Retention,
                        StateSpaceDuality)
from .latent import LatentAttention
from .feedforward import (FeedForward, SwiGLU, DenseMLP, RoutedExperts, GluMLP, SumFeedForward, TableExperts,
                          RowGatedFeedForward)
from .block import PreNormBlock, GatedSandwichBlock, ResidualGate, PostNormBlock, ParallelBlock
from .depth import DepthWeightedAverage
from .embedding import Embedding, OutputHead
from .model import DecoderModel, LayerCall

__all__ = ["Part", "StepContext", "StepPlan", "to_device_matrix", "to_device_vector", "linear", "RMSNorm",
           "LayerNorm", "RotaryTable", "Mixer", "GQAAttention", "GatedSinkAttention", "GatedLinearAttention",
           "ChannelDeltaRule", "FeedForward", "SwiGLU", "DenseMLP", "PreNormBlock", "GatedSandwichBlock", "ResidualGate",
           "ChunkedTalkingAttention", "ParallelMixers", "MatrixMemory", "ShiftedDecayRecurrence", "RoutedExperts", "PostNormBlock",
           "DepthWeightedAverage", "LatentAttention", "GluMLP", "SumFeedForward", "TableExperts",
           "Retention", "StateSpaceDuality", "RowGatedFeedForward", "ParallelBlock",
           "Embedding", "OutputHead", "DecoderModel", "LayerCall"]
