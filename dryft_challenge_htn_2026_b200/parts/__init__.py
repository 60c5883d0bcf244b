"""Parts a model is put together from: norms, position encodings, mixers, feed-forwards, blocks."""
from .base import ParamDecl, Part, Runtime, build_part, register_part
from . import norm, position, attention, attention_masked, linear_attention, gated_linear_attention, latent_attention, diff_attention, recurrence, parallel, feedforward, moe, block  # noqa: F401  (register the built-in parts)
from .attention import GQAAttention
from .attention_masked import MaskedAttention
from .block import PostNormBlock, PreNormBlock, SandwichBlock
from .feedforward import DenseMLP, GatedMLP
from .gated_linear_attention import GatedLinearAttention
from .latent_attention import LatentAttention
from .linear_attention import LinearAttention
from .moe import RoutedMLP
from .diff_attention import DiffAttention
from .norm import GroupRMSNorm, OnePlusRMSNorm, RMSNorm, ScalarRMSNorm
from .recurrence import LowerBoundRecurrence, StateSpace
from .parallel import ParallelMixer
from .position import RotaryHalf, RotaryPairs, RotaryPart, Sinusoid

__all__ = ["ParamDecl", "Part", "Runtime", "build_part", "register_part", "GQAAttention", "PreNormBlock", "GatedMLP",
           "RMSNorm", "RotaryHalf", "MaskedAttention", "LinearAttention", "ParallelMixer", "DenseMLP", "ScalarRMSNorm",
           "Sinusoid", "PostNormBlock", "GatedLinearAttention", "RoutedMLP", "OnePlusRMSNorm", "RotaryPart", "LatentAttention", "SandwichBlock", "RotaryPairs",
           "GroupRMSNorm", "DiffAttention", "LowerBoundRecurrence", "StateSpace"]
