from .model_config import (ConfigError, EndSpec, FeedForwardSpec, KeyReader, LayerSpec, MixerSpec,
                           ModelConfig, NormSpec, PositionSpec, RunEntry, pre_norm_layer,
                           read_config_json)
from .registry import (Architecture, architecture_name_of, get_architecture,
                       known_architectures, load_config, parse_config, register_architecture)
from .presets import SHAPES, shape
