from .model_config import (ConfigError, FeedForwardSpec, KeyReader, LayerSpec, MixerSpec,
                           ModelConfig, NormSpec, PositionSpec, RunEntry, read_config_json)
from .registry import (Architecture, architecture_name_of, get_architecture,
                       known_architectures, load_config, parse_config, register_architecture)
from .presets import SHAPES, shape
