from .model_config import ConfigError, LlamaConfig, read_config_json
from .nafevik_config import NafevikConfig
from .vatunex_config import VatunexConfig
from .zipelix_config import ZipelixConfig
from .pilutar_config import PilutarConfig
from .registry import Architecture, known_architectures, register_architecture, resolve_architecture

__all__ = ["ConfigError", "LlamaConfig", "NafevikConfig", "VatunexConfig", "ZipelixConfig", "PilutarConfig", "read_config_json", "Architecture",
           "known_architectures", "register_architecture", "resolve_architecture"]
