from .base import (Architecture, ConfigError, RawConfig, register_architecture, registered_architectures,
                   resolve_architecture)
from .qwen3 import Qwen3Config
from .vebonex import VebonexConfig
from .tikizen import TikizenConfig
from .sefalorn import SefalornConfig
