"""From a model folder (or a configuration and a seed) to a model with its weights on the device."""
from __future__ import annotations

import os
from typing import Any, Dict, Optional, Union

import torch

from ..config.registry import load_config, parse_config
from ..csrc.build import ensure_built
from ..weights.loader import SafetensorsSource, WeightStore, run_dtype_of
from ..weights.random_init import RandomSource, write_random_model


def _as_dtype(dtype: Union[str, torch.dtype]) -> torch.dtype:
    return dtype if isinstance(dtype, torch.dtype) else run_dtype_of(dtype)


def build_model(config_dict: Dict[str, Any], dtype: Union[str, torch.dtype]):
    """The model object (no weights yet) that config.json's architecture names."""
    from .. import models  # noqa: F401  (registers the built-in architectures)
    arch, cfg = parse_config(config_dict)
    return arch.model_class(cfg, _as_dtype(dtype))


def load_model(folder: str, dtype: Union[str, torch.dtype] = "bfloat16", device="cuda:0"):
    """Reads config.json and the safetensors of `folder`; the model class is chosen by config.json."""
    from .. import models  # noqa: F401
    if not os.path.isdir(folder):
        raise FileNotFoundError(f"model folder '{folder}' does not exist")
    arch, cfg = load_config(folder)
    model = arch.model_class(cfg, _as_dtype(dtype))
    ensure_built(model.kernels())
    source = SafetensorsSource(folder)
    try:
        store = WeightStore(source, model.weight_specs(), device, model.dtype, where=folder)
        model.bind(store)
    finally:
        source.close()
    return model


def random_model(config_dict: Dict[str, Any], seed: int, dtype: Union[str, torch.dtype] = "bfloat16",
                 device="cuda:0", std: float = 0.02):
    """A model with seeded random weights drawn on the device, without a folder in between; the same weights
    that write_random_folder writes for this configuration, seed and std."""
    model = build_model(config_dict, dtype)
    ensure_built(model.kernels())
    specs = model.weight_specs()
    store = WeightStore(RandomSource(specs, seed, std, torch.bfloat16), specs, device, model.dtype, where="random weights")
    model.bind(store)
    return model


def write_random_folder(folder: str, config_dict: Dict[str, Any], seed: int, std: float = 0.02,
                        dtype: torch.dtype = torch.bfloat16, fp32_names=(), device="cpu") -> None:
    """Writes config.json and model.safetensors with seeded random weights for a configuration: the tensors that
    random_model(config_dict, seed) holds.  `device`: where the values are drawn (the same values everywhere)."""
    model = build_model(config_dict, torch.float32)
    write_random_model(folder, model.config.to_dict() if hasattr(model.config, "to_dict") else config_dict,
                       model.weight_specs(), seed, std, dtype, fp32_names, device)
