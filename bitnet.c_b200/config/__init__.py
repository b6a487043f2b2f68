"""Typed configuration, the block-by-block model description, and the architecture registry."""
from .spec import (AttentionSpec, BlockSpec, ConfigError, GatedMlpSpec, LinearHeadSpec, ModelSpec, NoPositionSpec,
                   RmsNormSpec, RotarySpec, ScheduleEntry)
from .registry import (Architecture, architecture, architecture_of, known_architectures,
                       read_config_json, register_architecture, unregister_architecture)
from . import llama as _llama
from .llama import LlamaConfig

register_architecture(Architecture(
    name=_llama.ARCHITECTURE,
    read_config=LlamaConfig.from_dict,
    to_spec=LlamaConfig.to_spec,
    tensor_name=_llama.tensor_name,
    cap_positions=LlamaConfig.with_max_positions,
    config_to_dict=LlamaConfig.to_dict,
))

__all__ = [
    "AttentionSpec", "BlockSpec", "ConfigError", "GatedMlpSpec", "LinearHeadSpec", "ModelSpec", "NoPositionSpec",
    "RmsNormSpec", "RotarySpec", "ScheduleEntry", "Architecture", "architecture", "architecture_of",
    "known_architectures", "read_config_json", "register_architecture", "unregister_architecture",
    "LlamaConfig",
]
