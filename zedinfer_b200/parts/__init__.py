from .base import (Block, Embedding, FeedForward, Head, Mixer, Norm, Part, PositionEncoding, ResidualStream,
                   StepContext, block_class, build_part, register_block, register_embedding, register_feed_forward,
                   register_head, register_mixer, register_norm, register_position, unregister)
from . import attention, block, embedding, latent_attention, linear_recurrence, mlp, moe, rmsnorm, rope, ssm, tanhnorm  # noqa: F401  (registers the built-in kinds)
from .attention import AttentionMixer
from .block import BranchNormBlock, PreNormBlock, SandwichNormBlock
from .embedding import LearnedPositionEmbedding, OutputHead, ScaledTokenEmbedding, TokenEmbedding
from .linear_recurrence import ChannelDeltaMixer, ForgetGateMixer, GatedDeltaMixer, LightningMixer
from .latent_attention import LatentAttentionMixer
from .mlp import ClampedGatedMLP, GatedMLP, PolyNormMLP, SquaredReluMLP, TokenGatedTable
from .moe import RoutedExperts
from .rmsnorm import RMSNorm
from .tanhnorm import TanhNorm
from .rope import RotaryPosition, SpanRotaryPosition
from .ssm import Mamba2Mixer

__all__ = ["Block", "Embedding", "FeedForward", "Head", "Mixer", "Norm", "Part", "PositionEncoding", "ResidualStream",
           "StepContext", "block_class", "build_part", "register_block", "register_embedding",
           "register_feed_forward", "register_head", "register_mixer", "register_norm", "register_position", "unregister", "AttentionMixer", "PreNormBlock", "OutputHead",
           "TokenEmbedding", "GatedMLP", "RMSNorm", "RotaryPosition", "LearnedPositionEmbedding", "LatentAttentionMixer",
           "ClampedGatedMLP", "SquaredReluMLP", "RoutedExperts", "SpanRotaryPosition", "Mamba2Mixer", "BranchNormBlock",
           "ScaledTokenEmbedding", "ChannelDeltaMixer", "LightningMixer", "TokenGatedTable", "SandwichNormBlock", "ForgetGateMixer",
           "GatedDeltaMixer", "PolyNormMLP", "TanhNorm"]
