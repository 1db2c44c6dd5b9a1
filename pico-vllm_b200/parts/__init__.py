from .base import Param, Piece, Part, PagedKV, PagedTensors, PagedLatent, FixedState, CacheView, StepShape, MixerPlan
from .registry import register, make, MIXERS, FEED_FORWARDS, NORMS, POSITIONS
from .norm import RMSNorm, CentredNorm, NormedDelta, PassNorm, ScalarRMSNorm
from .rotary import Rotary, NoPosition, YarnRotary
from .attention import GQAAttention, QKNormAttention
from .linear_attention import DecayLinearAttention
from .latent_attention import LatentAttention
from .mlp import GatedMLP
from .moe import RoutedExperts
from .embedding import TokenEmbedding, OutputHead, LearnedPositions, TokenSideTable, TokenSideInput
from .conv_attention import ConvRopeAttention
from .delta_rule import GatedDeltaRule
from .norm import SumDelta
from .hyper import HyperConnection, HyperDelta, HyperBlock
from .recurrent import ExpGatedMatrixMemory, ForgetWriteLinearAttention, StateSpaceDuality
from .biased_attention import DistanceBiasAttention, ParallelMixers
from .block import PreNormBlock, SandwichBlock, ParallelBlock

__all__ = ["Param", "Piece", "Part", "PagedKV", "PagedTensors", "FixedState", "CacheView", "StepShape", "MixerPlan", "register", "make", "MIXERS",
           "FEED_FORWARDS", "NORMS", "POSITIONS", "RMSNorm", "Rotary", "NoPosition", "GQAAttention",
           "GatedMLP", "TokenEmbedding", "OutputHead", "PreNormBlock", "PagedLatent", "CentredNorm", "NormedDelta",
           "LatentAttention", "RoutedExperts", "SandwichBlock", "PassNorm", "YarnRotary", "QKNormAttention",
           "DecayLinearAttention", "ScalarRMSNorm", "LearnedPositions", "HyperConnection", "HyperDelta", "HyperBlock",
           "ExpGatedMatrixMemory", "ForgetWriteLinearAttention", "StateSpaceDuality", "DistanceBiasAttention", "ParallelMixers",
           "TokenSideTable", "TokenSideInput", "ConvRopeAttention", "GatedDeltaRule", "SumDelta", "ParallelBlock"]
