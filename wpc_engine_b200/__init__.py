"""A small, whole inference library for the Qwen2 dense decoder on one B200 (sm_100a).

    from wpc_engine_b200 import Engine, GenerationOptions, generate
    engine = Engine.from_folder("model_dir", dtype="bfloat16")
    ids = generate(engine, [[1, 2, 3], [4, 5]], GenerationOptions(max_tokens=16))

Layout: config/ (typed configurations), registry.py (architecture name -> model), weights/
(safetensors by tensor name, random-weights mode), parts/ (norm, position encoding, mixer,
feed-forward, block), models/ (a decoder as data, and the Qwen2 builder), cache/ (slots, pages,
per-sequence state), engine/ (the step function and the generation loop), sampling/, ops.py
(the Python face of the kernels) and csrc/ (the CUDA sources and their in-tree build).
"""
from .cache import CacheError
from .config import ConfigError, Qwen2Config
from .engine import Engine, GenerationOptions, SequenceStep, generate
from .ops import KernelError
from .registry import architecture_names, register_architecture, resolve, unregister_architecture
from .weights import WeightError, write_random_model

__all__ = ["CacheError", "ConfigError", "Engine", "GenerationOptions", "KernelError", "Qwen2Config",
           "SequenceStep", "WeightError", "architecture_names", "generate", "register_architecture",
           "resolve", "unregister_architecture", "write_random_model"]
