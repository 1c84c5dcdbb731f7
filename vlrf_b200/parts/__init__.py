from .block import PreNormBlock, SublayerNormBlock
from .context import StepContext, Workspace
from .embedding import LMHead, TokenEmbedding
from .feed_forward import DenseMLP
from .latent_attention import LatentAttention
from .mixer import CausalSelfAttention
from .moe import RoutedExperts
from .norm import GroupRMSNorm, LayerNorm
from .position import LearnedAbsolutePositions, RotaryPositions
from .registry import get_part, part_names, register_part, unregister_part

__all__ = ["PreNormBlock", "SublayerNormBlock", "LatentAttention", "RoutedExperts", "GroupRMSNorm", "RotaryPositions", "StepContext", "Workspace", "LMHead", "TokenEmbedding", "DenseMLP",
           "CausalSelfAttention", "LayerNorm", "LearnedAbsolutePositions", "get_part", "part_names",
           "register_part", "unregister_part"]
