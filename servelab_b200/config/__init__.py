"""Typed configuration: model specs as data, family configs, engine knobs."""

from .engine import CacheConfig, EngineConfig, SchedulerConfig
from .daferax import DaferaxConfig
from .dezelorn import DezelornConfig
from .qwen2 import ConfigError, Qwen2Config
from .sumolorn import SumolornConfig
from .zimupel import ZimupelConfig
from .registry import (config_from_dict, load_config, model_spec_from_config,
                       register_architecture, registered_architectures,
                       resolve_architecture)
from .specs import (AttentionSpec, BlockSpec, ConvTalkAttentionSpec, DecayAttentionSpec,
                    DifferentialAttentionSpec, DynamicTanhSpec, GatedMLPSpec,
                    LatentAttentionSpec, LayerNormSpec, LayerRun, ModelSpec, NoPositionSpec,
                    NormedAttentionSpec, PairRotarySpec, ParallelMixersSpec, PartSpec, RMSNormSpec,
                    RotarySpec, RoutedExpertsSpec)

register_architecture(Qwen2Config.architecture, Qwen2Config, model_type=Qwen2Config.model_type)
register_architecture(DezelornConfig.architecture, DezelornConfig, model_type=DezelornConfig.model_type)
register_architecture(DaferaxConfig.architecture, DaferaxConfig, model_type=DaferaxConfig.model_type)
register_architecture(ZimupelConfig.architecture, ZimupelConfig, model_type=ZimupelConfig.model_type)
register_architecture(SumolornConfig.architecture, SumolornConfig, model_type=SumolornConfig.model_type)

__all__ = [
    "AttentionSpec", "BlockSpec", "CacheConfig", "ConfigError", "ConvTalkAttentionSpec",
    "DaferaxConfig", "DecayAttentionSpec", "DezelornConfig", "DifferentialAttentionSpec", "DynamicTanhSpec",
    "EngineConfig",
    "GatedMLPSpec", "LatentAttentionSpec", "LayerNormSpec", "LayerRun", "ModelSpec", "NoPositionSpec",
    "NormedAttentionSpec", "PairRotarySpec", "ParallelMixersSpec", "PartSpec",
    "Qwen2Config", "RMSNormSpec", "RotarySpec", "RoutedExpertsSpec", "SchedulerConfig", "SumolornConfig", "ZimupelConfig",
    "config_from_dict", "load_config", "model_spec_from_config",
    "register_architecture", "registered_architectures", "resolve_architecture",
]
