"""The random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed, and the same distribution drawn directly on the device for sizes
that should not pass through a file.

Matrices, tables and biases are N(0, 0.02); norm gains are 1 + N(0, 0.02), so that no gain
is near zero.  The reference has no such mode.  Folder mode draws on the host with a seeded
generator, tensor by tensor in the model's own order, so a folder is reproducible from
(configuration, seed, dtype) alone.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from .. import ops
from .loader import bind_model, device_dtype
from .safetensors_io import write_safetensors

STD = 0.02


def _name_seed(seed: int, name: str) -> int:
    h = 1469598103934665603
    for ch in name.encode("utf-8"):
        h = ((h ^ ch) * 1099511628211) & ((1 << 64) - 1)
    return (h ^ (seed * 0x9E3779B97F4A7C15)) & ((1 << 63) - 1)


def _random_index(spec, seed: int, name: str) -> torch.Tensor:
    """An integer table: int32 drawn evenly from 0 .. spec.high - 1 on the host (zeros without `high`)."""
    if not spec.high:
        return torch.zeros(spec.shape, dtype=torch.int32)
    gen = torch.Generator(device="cpu")
    gen.manual_seed(_name_seed(seed, name))
    return torch.randint(0, int(spec.high), spec.shape, generator=gen, dtype=torch.int32)


def write_random_model(folder: str, config, seed: int, dtype: torch.dtype = torch.bfloat16) -> str:
    """Writes config.json and model.safetensors for `config` (a registered architecture's
    configuration object); returns the folder."""
    from ..registry import resolve
    raw = config.to_dict()
    model = resolve(raw).build(config)
    os.makedirs(folder, exist_ok=True)
    tensors = []
    for name, (_, _, spec) in model.wanted_tensors().items():
        if spec.kind == "index":
            tensors.append((name, _random_index(spec, seed, name)))
            continue
        gen = torch.Generator(device="cpu")
        gen.manual_seed(_name_seed(seed, name))
        t = torch.randn(spec.shape, generator=gen, dtype=torch.float32) * STD
        if spec.init == "gain":
            t = t + 1.0
        tensors.append((name, t.to(dtype)))
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f, indent=1)
    return folder


def random_weights_on_device(model, seed: int, dtype: torch.dtype, device) -> None:
    """Fills the model's tensors on the device with the fill kernel (no file, no host copy)."""
    tensors: Dict[str, torch.Tensor] = {}
    for name, (_, _, spec) in model.wanted_tensors().items():
        if spec.kind == "index":          # small tables of integers: drawn on the host
            tensors[name] = _random_index(spec, seed, name).to(device)
            continue
        t = torch.empty(spec.shape, dtype=device_dtype(dtype, spec.kind, dtype), device=device)
        ops.fill_normal(t, _name_seed(seed, name), 1.0 if spec.init == "gain" else 0.0, STD)
        tensors[name] = t
    bind_model(model, tensors)
