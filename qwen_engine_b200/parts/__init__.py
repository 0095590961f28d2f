from .base import (Arena, Block, FeedForward, GroupStepView, Mixer, Norm, Part, PartSpec,
                   PositionEncoding, StepContext, register, NORMS, POSITION_ENCODINGS, MIXERS,
                   FEED_FORWARDS, BLOCKS)
from .norm import GroupRMSNorm, RMSNorm
from .rope import NeoxRope, ScaledRope
from .attention import GQAAttention
from .linear_attention import DecayedLinearAttention, GatedLinearAttention
from .latent_attention import LatentAttention
from .delta_rule import GatedDeltaRule
from .moe import RoutedExperts
from .parallel import ParallelMixers
from .mlp import SwiGLU
from .block import PreNormBlock
from .gated_post_norm import GatedPostNormBlock
from .sandwich_norm import SandwichNormBlock

__all__ = ["Arena", "Block", "FeedForward", "GroupStepView", "Mixer", "Norm", "Part", "PartSpec",
           "PositionEncoding", "StepContext", "register", "NORMS", "POSITION_ENCODINGS", "MIXERS",
           "FEED_FORWARDS", "BLOCKS", "RMSNorm", "GroupRMSNorm", "NeoxRope", "ScaledRope", "GQAAttention", "GatedLinearAttention", "DecayedLinearAttention", "LatentAttention", "GatedDeltaRule", "RoutedExperts", "ParallelMixers", "SwiGLU",
           "PreNormBlock", "GatedPostNormBlock", "SandwichNormBlock"]
