"""Sampling: greedy, banned ids, temperature.  The device kernel is `ops.sample`; this module
holds what the host needs around it."""
from .sampler import banned_from_env, stop_ids_of_folder, uniform_for

__all__ = ["banned_from_env", "stop_ids_of_folder", "uniform_for"]
