from .fields import read_config_dict, required, optional
from .mabedra import MabedraConfig
from .qwen3 import Qwen3Config
from .ropulix import RopulixConfig
from .sorulix import SorulixConfig
from .tafisun import TafisunConfig
from .registry import (
    Architecture,
    architecture_for,
    load_config,
    register_architecture,
    registered_architectures,
)

__all__ = [
    "Architecture",
    "MabedraConfig",
    "Qwen3Config",
    "RopulixConfig",
    "SorulixConfig",
    "TafisunConfig",
    "architecture_for",
    "load_config",
    "optional",
    "read_config_dict",
    "register_architecture",
    "registered_architectures",
    "required",
]
