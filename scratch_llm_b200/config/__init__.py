"""Typed configurations and the architecture registry."""

from .llama import LlamaConfig
from .registry import (ARCHITECTURES, Architecture, config_from_dict, get_architecture,
                       load_config, register_architecture, save_config)
from .spec import LayerSpec, ModelSpec, PartSpec, Run, sequential_order, standard_layer

register_architecture("LlamaForCausalLM", LlamaConfig)

__all__ = ["ARCHITECTURES", "Architecture", "LayerSpec", "LlamaConfig", "ModelSpec", "standard_layer",
           "PartSpec", "Run", "config_from_dict", "get_architecture", "load_config",
           "register_architecture", "save_config", "sequential_order"]
