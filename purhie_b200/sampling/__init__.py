"""Sampling: greedy, temperature, top-k, top-p, min-p and penalties, in the reference's order."""
from .mt19937_64 import MT19937_64
from .sampler import LOGIT_RANGE, Sampler, SamplerParams

__all__ = ["MT19937_64", "Sampler", "SamplerParams", "LOGIT_RANGE"]
