"""Configuration: typed per-architecture classes and the specs they produce."""
from .registry import (architectures, config_class, config_from_dict, load_config,
                       register_architecture)
from .specs import (AttentionSpec, BlockSpec, DenseMlpSpec, EmbeddingSpec, FeedForwardSpec, GatedDeltaSpec,
                    GatedLinearAttentionSpec,
                    GatedMlpSpec, LatentAttentionSpec, MixerSpec, ModelSpec, NormSpec, OutputSpec, PositionSpec,
                    RoutedExpertsSpec, ScheduleEntry, StreamInjection, MixerPairSpec, RetentionSpec, TokenSideSpec)
from .qwen3 import Qwen3Config
from .romepel import RomepelConfig
from .zevivik import ZevivikConfig
from .pikalorn import PikalornConfig
from .vodalorn import VodalornConfig

__all__ = [
    "architectures", "config_class", "config_from_dict", "load_config", "register_architecture",
    "AttentionSpec", "BlockSpec", "EmbeddingSpec", "FeedForwardSpec", "GatedMlpSpec", "MixerSpec",
    "ModelSpec", "NormSpec", "OutputSpec", "PositionSpec", "ScheduleEntry", "Qwen3Config", "RomepelConfig",
    "DenseMlpSpec", "GatedLinearAttentionSpec", "LatentAttentionSpec", "RoutedExpertsSpec", "StreamInjection",
    "ZevivikConfig", "GatedDeltaSpec", "PikalornConfig", "MixerPairSpec", "RetentionSpec", "TokenSideSpec",
    "VodalornConfig",
]
