"""A small B200-native model library with generation of its own.

Everything between a request's tokens and its next token for the Qwen2 MoE sparse decoder:
configuration and registry (config/), weights (weights/), parts and models (parts/, models/),
the paged cache (cache/), the step function and the generation loop (engine/), sampling
(sampling/), and hand-written sm_100a kernels (csrc/, kernels/).
"""
from .config import ConfigError, Qwen2MoeConfig, register_architecture, registered_architectures
from .weights import WeightError, WeightSpec
from . import models  # registers the built-in architectures
from .engine import Engine, StepEntry, StepError, build_model, load_model, random_model, write_random_folder
from .engine.generate import GenParams, GenResult, GenStats, generate, plan_batches
from .sampling import Sampler
from .model import Model

__version__ = "0.1.0"
