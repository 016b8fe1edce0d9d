"""Registers the built-in parts."""
from .attention import AttentionMixer
from .base import register_part
from .block import HyperConnectionBlock, OutputNormResidualBlock, ParallelResidualBlock, PreNormResidualBlock
from .delta_rule import GatedDeltaRule
from .embedding import LinearHead, TokenEmbedding
from .feedforward import DenseFeedForward, SwiGLU
from .latent_attention import LatentAttention
from .linear_attention import DecayLinearAttention
from .mamba2 import Mamba2Mixer
from .mlstm import MatrixMemory
from .moe import RoutedExperts
from .norm import RMSNorm
from .position import NoPosition, RotaryInterleaved, RotaryNeox
from .shortconv import ShortConvMixer
from .sidebyside import SideBySideMixer
from .streamop import StretchEntry

register_part("mixer", "attention", AttentionMixer, replace=True)
register_part("mixer", "short_conv", ShortConvMixer, replace=True)
register_part("feed_forward", "swiglu", SwiGLU, replace=True)
register_part("norm", "rmsnorm", RMSNorm, replace=True)
register_part("position", "rope_neox", RotaryNeox, replace=True)
register_part("position", "none", NoPosition, replace=True)
register_part("block", "prenorm_residual", PreNormResidualBlock, replace=True)
register_part("embedding", "token_table", TokenEmbedding, replace=True)
register_part("head", "linear", LinearHead, replace=True)
register_part("mixer", "decay_linear_attention", DecayLinearAttention, replace=True)
register_part("mixer", "side_by_side", SideBySideMixer, replace=True)
register_part("feed_forward", "dense", DenseFeedForward, replace=True)
register_part("position", "rope_interleaved", RotaryInterleaved, replace=True)
register_part("block", "parallel_residual", ParallelResidualBlock, replace=True)
register_part("stream_op", "stretch_entry", StretchEntry, replace=True)
register_part("block", "outnorm_residual", OutputNormResidualBlock, replace=True)
register_part("mixer", "mamba2", Mamba2Mixer, replace=True)
register_part("feed_forward", "routed_experts", RoutedExperts, replace=True)
register_part("block", "hyper_connections", HyperConnectionBlock, replace=True)
register_part("mixer", "latent_attention", LatentAttention, replace=True)
register_part("mixer", "gated_delta_rule", GatedDeltaRule, replace=True)
register_part("mixer", "matrix_memory", MatrixMemory, replace=True)
