from .decoder import DecoderModel, LayerCall, Binding
from .qwen2 import build_qwen2
from .zapipel import build_zapipel
from .zikupel import build_zikupel
from .zazilix import build_zazilix

__all__ = ["DecoderModel", "LayerCall", "Binding", "build_qwen2", "build_zapipel", "build_zikupel", "build_zazilix"]
