"""Typed configuration: part specifications, the model specification built from them, and the
architecture's own config.json reader."""
from .specs import (AttentionSpec, DenseMLPSpec, GatedLinearAttentionSpec, GatedMLPSpec, LayerSpec, LinearAttentionSpec,
                    MaskedAttentionSpec, ModelSpec, OnePlusRMSNormSpec, ParallelMixerSpec, PostNormLayerSpec, RMSNormSpec,
                    RotaryHalfSpec, RotaryPairsSpec, RotaryPartSpec, RoutedMLPSpec, SandwichLayerSpec, ScalarRMSNormSpec, ScheduleEntry,
                    SinusoidSpec, UnitRMSNormSpec, LatentAttentionSpec, DiffAttentionSpec, GroupRMSNormSpec,
                    LowerBoundRecurrenceSpec, StateSpaceSpec)
from .base import ConfigError, ModelConfig
from .nevotar import NevotarConfig
from .nilivik import NilivikConfig
from .pibulix import PibulixConfig
from .qwen3 import Qwen3Config
from .venidra import VenidraConfig

__all__ = ["AttentionSpec", "DenseMLPSpec", "GatedMLPSpec", "LayerSpec", "LinearAttentionSpec", "MaskedAttentionSpec",
           "ModelSpec", "ParallelMixerSpec", "RMSNormSpec", "RotaryHalfSpec", "ScalarRMSNormSpec", "ScheduleEntry",
           "SinusoidSpec", "ConfigError", "ModelConfig", "NilivikConfig", "Qwen3Config", "PibulixConfig",
           "GatedLinearAttentionSpec", "OnePlusRMSNormSpec", "PostNormLayerSpec", "RotaryPartSpec", "RoutedMLPSpec", "VenidraConfig", "LatentAttentionSpec", "RotaryPairsSpec",
           "SandwichLayerSpec", "UnitRMSNormSpec", "NevotarConfig", "DiffAttentionSpec", "GroupRMSNormSpec",
           "LowerBoundRecurrenceSpec", "StateSpaceSpec"]
