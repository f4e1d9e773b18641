"""Sampling: greedy, temperature, top-p."""
from .sampler import Sampler, uniforms_for
