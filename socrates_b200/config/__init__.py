from .plan import LayerSpec, ModelPlan, PartSpec, RunEntry
from .qwen3 import ConfigError, Qwen3Config
from .bofusun import BofusunConfig
from .loletar import LoletarConfig
from .samerax import SameraxConfig
from .magedra import MagedraConfig
from .registry import (config_from_dict, known_architectures, load_config,
                       register_architecture, unregister_architecture)
from .engine import EngineConfig

__all__ = [
    "LayerSpec", "ModelPlan", "PartSpec", "RunEntry", "ConfigError", "Qwen3Config", "BofusunConfig", "LoletarConfig", "SameraxConfig", "MagedraConfig",
    "config_from_dict", "known_architectures", "load_config", "register_architecture",
    "unregister_architecture", "EngineConfig",
]
