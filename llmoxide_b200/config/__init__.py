"""Typed configuration, the architecture registry and the part-level model
description that the rest of the package reads."""

from .qwen3 import Qwen3Config
from .registry import architectures, config_class, read_config, register_architecture
from .fusasun import FusasunConfig
from .ninenex import NinenexConfig
from .tifapel import TifapelConfig
from .voserax import VoseraxConfig
from .spec import BlockSpec, LayerCall, ModelSpec, PartSpec, TensorSpec, default_schedule

register_architecture("Qwen3ForCausalLM", Qwen3Config)
register_architecture("Tifapel", TifapelConfig)
register_architecture("Voserax", VoseraxConfig)
register_architecture("Ninenex", NinenexConfig)
register_architecture("Fusasun", FusasunConfig)

__all__ = [
    "Qwen3Config", "FusasunConfig", "NinenexConfig", "TifapelConfig", "VoseraxConfig", "architectures", "config_class", "read_config", "register_architecture",
    "BlockSpec", "LayerCall", "ModelSpec", "PartSpec", "TensorSpec", "default_schedule",
]
