"""Greedy and seeded sampling as the reference defines them."""
from .params import MAX_PENALTY_WINDOW, Sampling
from .sampler import Sampler, pack_params

__all__ = ["MAX_PENALTY_WINDOW", "Sampling", "Sampler", "pack_params"]
