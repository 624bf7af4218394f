"""Configuration: typed architecture configs, the model spec they produce, the registry."""

from .dapozen import ARCHITECTURE as DAPOZEN_ARCHITECTURE
from .dapozen import DapozenConfig
from .digosun import ARCHITECTURE as DIGOSUN_ARCHITECTURE
from .digosun import DigosunConfig
from .gikarax import ARCHITECTURE as GIKARAX_ARCHITECTURE
from .gikarax import GikaraxConfig
from .poselorn import ARCHITECTURE as POSELORN_ARCHITECTURE
from .poselorn import PoselornConfig
from .qwen2 import ARCHITECTURE as QWEN2_ARCHITECTURE
from .qwen2 import ConfigError, Qwen2Config
from .registry import (config_class_for, load_config, register_architecture,
                       supported_architectures, unregister_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, RunSpec

register_architecture(QWEN2_ARCHITECTURE, Qwen2Config)
register_architecture(DIGOSUN_ARCHITECTURE, DigosunConfig)
register_architecture(DAPOZEN_ARCHITECTURE, DapozenConfig)
register_architecture(POSELORN_ARCHITECTURE, PoselornConfig)
register_architecture(GIKARAX_ARCHITECTURE, GikaraxConfig)

__all__ = ["ConfigError", "Qwen2Config", "QWEN2_ARCHITECTURE", "DigosunConfig",
           "DIGOSUN_ARCHITECTURE", "DapozenConfig", "DAPOZEN_ARCHITECTURE", "PoselornConfig",
           "POSELORN_ARCHITECTURE", "GikaraxConfig", "GIKARAX_ARCHITECTURE", "LayerSpec", "ModelSpec",
           "PartSpec", "RunSpec", "config_class_for", "load_config",
           "register_architecture", "supported_architectures", "unregister_architecture"]
