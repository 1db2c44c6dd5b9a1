from .base import KeyReader, read_config_json, architecture_name
from .qwen2 import Qwen2Config
from .zapipel import ZapipelConfig
from .zikupel import ZikupelConfig
from .zazilix import ZazilixConfig
from .engine import EngineConfig, canonical_dtype

__all__ = ["KeyReader", "read_config_json", "architecture_name", "Qwen2Config", "ZapipelConfig", "ZikupelConfig", "ZazilixConfig", "EngineConfig",
           "canonical_dtype"]
