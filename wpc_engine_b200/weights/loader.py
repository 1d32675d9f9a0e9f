"""Weights by tensor name: from a model folder onto the device, checked as a whole.

Every tensor that the model's parts want is looked up by its stored name
(wpc-runtime/src/model.rs:70, 80-94, 114).  Where the reference panics at the first missing
tensor (weights.rs:145, 151) and compares element counts only (weights.rs:44-47), this loader
collects everything that is wrong (missing, unexpected, wrong shape, unusable dtype) and
raises one `WeightError` that lists it all.

Types: a matrix or table stays as stored (bfloat16 stays bfloat16, a 32-bit tensor stays
32-bit; float16 is widened to float32, which is exact); vectors (gains, biases) are widened to
float32; integer tables (kind "index") become int32.  With `dtype=float32` everything is widened to float32 (the reference's own
behaviour, weights.rs:153-173).
"""
from __future__ import annotations

import sys
from typing import Dict, List

import torch

from ..parts.base import Part
from .safetensors_io import ModelFiles

_FLOATS = ("F32", "F16", "BF16")
_INTS = ("I32", "I64")


class WeightError(RuntimeError):
    """The tensors of a model folder do not fit the model; lists every problem."""

    def __init__(self, missing: List[str], unexpected: List[str], wrong_shape: List[str], wrong_dtype: List[str]):
        self.missing, self.unexpected = missing, unexpected
        self.wrong_shape, self.wrong_dtype = wrong_shape, wrong_dtype
        lines = []
        for title, items in (("missing tensors", missing), ("unexpected tensors", unexpected),
                             ("wrong shapes", wrong_shape), ("unusable dtypes", wrong_dtype)):
            if items:
                lines.append(f"{title} ({len(items)}):")
                lines += [f"  {it}" for it in items]
        super().__init__("the weights do not fit the model\n" + "\n".join(lines))


def check_names(wanted: Dict[str, object], files: ModelFiles, ignored=()) -> None:
    have = set(files.names())
    missing = sorted(n for n in wanted if n not in have)
    unexpected = sorted(n for n in have if n not in wanted and n not in ignored)
    wrong_shape, wrong_dtype = [], []
    for name, (_, _, spec) in wanted.items():
        if name not in have:
            continue
        if tuple(files.shape(name)) != tuple(spec.shape):
            wrong_shape.append(f"{name}: stored {list(files.shape(name))}, the model wants {list(spec.shape)}")
        accepted = _INTS if spec.kind == "index" else _FLOATS
        if files.dtype_name(name) not in accepted:
            wrong_dtype.append(f"{name}: stored as {files.dtype_name(name)}, wanted one of {', '.join(accepted)}")
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(missing, unexpected, wrong_shape, wrong_dtype)


def device_dtype(stored: torch.dtype, kind: str, dtype: torch.dtype) -> torch.dtype:
    """The type in which a tensor of `kind`, stored as `stored`, is kept for a model that
    computes in `dtype`."""
    if kind == "index":
        return torch.int32           # integer tables are kept as int32 whatever the model's type
    if dtype == torch.float32 or kind == "vector":
        return torch.float32
    if stored == torch.bfloat16:
        return torch.bfloat16
    return torch.float32             # stored in 32 bits: stays so; float16 widens exactly


def finalize_parts(part: Part) -> None:
    for sub in part.subparts().values():
        finalize_parts(sub)
    fin = getattr(part, "finalize", None)
    if fin is not None:
        fin()


def bind_model(model, tensors: Dict[str, torch.Tensor]) -> None:
    """Hands each part its tensors (already on the device, right type) and lets parts fuse."""
    wanted = model.wanted_tensors()
    per_part: Dict[int, Dict[str, torch.Tensor]] = {}
    owners: Dict[int, Part] = {}
    for name, (part, local, _) in wanted.items():
        per_part.setdefault(id(part), {})[local] = tensors[name]
        owners[id(part)] = part
    for pid, part in owners.items():
        part.bind(per_part[pid])
    for _, root in model.roots():
        finalize_parts(root)


def load_weights(model, folder: str, dtype: torch.dtype, device) -> None:
    files = ModelFiles(folder)
    try:
        wanted = model.wanted_tensors()
        check_names(wanted, files, ignored=model.ignored)
        tensors = {}
        wide = []
        for name, (_, _, spec) in wanted.items():
            host = files.read(name)
            kept = device_dtype(host.dtype, spec.kind, dtype)
            if dtype == torch.bfloat16 and kept == torch.float32 and spec.kind in ("matrix", "table"):
                wide.append(name)
            tensors[name] = host.to(device=device, dtype=kept).contiguous()
    finally:
        files.close()
    if wide:
        # nothing is converted behind the user's back; the slow path is named once instead
        print(f"[wpc_engine_b200] {len(wide)} matrices of {folder} are stored in 32 or 16-bit IEEE floats "
              f"(first: {wide[0]}) and stay float32: their products run on the CUDA cores, not on the tensor "
              "cores.  Store the checkpoint in bfloat16 for the fast path.", file=sys.stderr, flush=True)
    bind_model(model, tensors)
