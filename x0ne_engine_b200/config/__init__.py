"""Typed configurations and the architecture registry."""
from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry
from .registry import (architectures, config_from_dict, config_from_folder, detect,
                       register_architecture, spec_from_folder, unregister_architecture)
from .qwen3 import ARCHITECTURE as _QWEN3, MODEL_TYPE as _QWEN3_TYPE, Qwen3Config
from .rovurax import ARCHITECTURE as _ROVURAX, MODEL_TYPE as _ROVURAX_TYPE, RovuraxConfig

from .tenetar import ARCHITECTURE as _TENETAR, MODEL_TYPE as _TENETAR_TYPE, TenetarConfig

from .retuvik import ARCHITECTURE as _RETUVIK, MODEL_TYPE as _RETUVIK_TYPE, RetuvikConfig

from .barorax import ARCHITECTURE as _BARORAX, MODEL_TYPE as _BARORAX_TYPE, BaroraxConfig

register_architecture(_QWEN3, _QWEN3_TYPE, Qwen3Config)
register_architecture(_TENETAR, _TENETAR_TYPE, TenetarConfig)
register_architecture(_ROVURAX, _ROVURAX_TYPE, RovuraxConfig)
register_architecture(_RETUVIK, _RETUVIK_TYPE, RetuvikConfig)
register_architecture(_BARORAX, _BARORAX_TYPE, BaroraxConfig)

__all__ = ["ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "RunEntry", "Qwen3Config", "RovuraxConfig", "TenetarConfig", "RetuvikConfig", "BaroraxConfig",
           "architectures", "config_from_dict", "config_from_folder", "detect",
           "register_architecture", "spec_from_folder", "unregister_architecture"]
