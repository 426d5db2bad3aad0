from .model_config import LlamaConfig, RopeScaling, read_config_json, write_config_json
from .rotepel_config import RotepelConfig, RotepelLayer
from .lomopel_config import GatedDeltaConfig, LomopelConfig, LomopelLayer, SoftmaxMixerConfig
from .bufulorn_config import BufulornConfig, BufulornLayer, ChunkAttentionConfig, FeedForwardConfig, HeadDecayDeltaConfig
from .pironex_config import (ClampedExpertsConfig, PironexConfig, PironexLayer, PooledAttentionConfig, StateSpaceConfig,
                             WindowLatentConfig)
from .engine_config import EngineConfig, parse_dtype
from .registry import (Architecture, register_architecture, unregister_architecture,
                       known_architectures, architecture_for)

__all__ = ["LlamaConfig", "RopeScaling", "RotepelConfig", "RotepelLayer", "LomopelConfig", "LomopelLayer", "SoftmaxMixerConfig",
           "GatedDeltaConfig", "BufulornConfig", "BufulornLayer", "ChunkAttentionConfig", "FeedForwardConfig",
           "HeadDecayDeltaConfig", "PironexConfig", "PironexLayer", "PooledAttentionConfig", "StateSpaceConfig",
           "WindowLatentConfig", "ClampedExpertsConfig", "read_config_json", "write_config_json", "EngineConfig",
           "parse_dtype", "Architecture", "register_architecture", "unregister_architecture",
           "known_architectures", "architecture_for"]
