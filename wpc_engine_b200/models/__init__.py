from .decoder import DecoderModel, Run
from .qwen2 import build_qwen2

__all__ = ["DecoderModel", "Run", "build_qwen2"]
