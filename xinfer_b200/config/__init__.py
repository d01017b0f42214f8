"""Configuration: typed per-architecture configs, part specs and the architecture registry."""
from .plan import (AttentionSpec, BlockOp, BlockSpec, FeedForwardSpec, LayerRun, ModelPlan, NormSpec,
                   PartSpec, RopeSpec, pre_norm_block)
from .errors import ConfigError
from .qwen3 import Qwen3Config
from .registry import (ArchitectureEntry, architecture_entry, config_from_dict,
                       known_architectures, load_config, read_config_json,
                       register_architecture, unregister_architecture)
from .engine import EngineConfig
from .generation import GenerationConfig

__all__ = [
    "AttentionSpec", "BlockOp", "BlockSpec", "pre_norm_block", "FeedForwardSpec", "LayerRun", "ModelPlan", "NormSpec",
    "PartSpec", "RopeSpec", "ConfigError", "Qwen3Config", "ArchitectureEntry",
    "architecture_entry", "config_from_dict", "known_architectures", "load_config",
    "read_config_json", "register_architecture", "unregister_architecture", "EngineConfig", "GenerationConfig",
]
