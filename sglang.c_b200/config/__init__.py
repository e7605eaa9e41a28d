from .base import ConfigError, read_config_json
from .buborax import BuboraxConfig, BuboraxLayer
from .gpt2 import GPT2Config
from .lubavik import LubavikConfig, LubavikLayer
from .tukavik import TukavikConfig, TukavikLayer
from .zuretar import ZuretarConfig, ZuretarLayer
from .registry import (Architecture, known_architectures, load_config,
                       register_architecture, resolve_architecture)

__all__ = ["ConfigError", "read_config_json", "BuboraxConfig", "BuboraxLayer", "GPT2Config", "LubavikConfig", "LubavikLayer", "TukavikConfig", "TukavikLayer", "ZuretarConfig", "ZuretarLayer", "Architecture",
           "known_architectures", "load_config", "register_architecture",
           "resolve_architecture"]
