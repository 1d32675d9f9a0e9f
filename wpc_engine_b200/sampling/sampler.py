"""Host side of sampling.

Greedy picking takes the first strictly greatest logit and skips banned ids
(wpc-runtime/src/sampling.rs:3-13, 35-51); the banned list may come from the environment
variable WPC_BAN_TOKENS (sampling.rs:23-31).  Temperature sampling is not in the reference:
p = softmax(logits / T) in float32, one uniform number per drawn token from a counter-based
generator keyed by (seed, request number, tokens drawn so far), so that a request draws the
same numbers alone or in any batch, and the first index whose cumulative probability exceeds
it is taken.
"""
from __future__ import annotations

import json
import os
from typing import List

_M64 = (1 << 64) - 1


def _mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def uniform_for(seed: int, request: int, step: int) -> float:
    """The number in [0, 1) that the device sampler draws; the kernel computes the same."""
    z = _mix64(seed & _M64)
    z = _mix64(z ^ (request & _M64))
    z = _mix64(z ^ (step & _M64))
    return (z >> 40) * (1.0 / (1 << 24))


def banned_from_env(name: str = "WPC_BAN_TOKENS") -> List[int]:
    """Comma-separated ids; entries that are not numbers are skipped (sampling.rs:23-31)."""
    out = []
    for part in os.environ.get(name, "").split(","):
        part = part.strip()
        if part.isdigit():
            out.append(int(part))
    return out


def stop_ids_of_folder(folder: str) -> List[int]:
    """`eos_token_id` (a number or a list) of generation_config.json and of config.json,
    united, sorted, without doubles (wpc-runtime/src/main.rs:449-488)."""
    ids = set()
    for name in ("generation_config.json", "config.json"):
        try:
            with open(os.path.join(folder, name)) as f:
                raw = json.load(f)
        except (OSError, json.JSONDecodeError):
            continue
        eos = raw.get("eos_token_id") if isinstance(raw, dict) else None
        if isinstance(eos, int) and not isinstance(eos, bool) and eos >= 0:
            ids.add(eos)
        elif isinstance(eos, list):
            ids.update(e for e in eos if isinstance(e, int) and not isinstance(e, bool) and e >= 0)
    return sorted(ids)
