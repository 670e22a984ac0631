from .base import (ConfigError, FeedForwardSpec, LayerSpec, MixerSpec, ModelConfig, ModelSpec,
                   NormSpec, PositionSpec, config_from_dict, load_config, register_architecture,
                   registered_architectures)
