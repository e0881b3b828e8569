"""From a model folder to a model on the device."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .models.model import Model
from .ops.ops import Ops
from .registry import Architecture, load_config
from .weights.loader import load_checkpoint

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name in (torch.bfloat16, torch.float32):
            return name
        raise ValueError(f"dtype {name} is not built; known: bfloat16, float32")
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype '{name}' is not built; known: bfloat16, float32") from None


def build_model(arch: Architecture, config, dtype: torch.dtype, device="cuda:0") -> Model:
    return Model(arch.model_spec(config), Ops(dtype, device))


def load_model(model_dir: str, dtype="bfloat16", device="cuda:0") -> Tuple[Architecture, object, Model]:
    """(architecture, typed configuration, model with its weights on the device)."""
    dtype = parse_dtype(dtype)
    arch, config = load_config(model_dir)
    model = build_model(arch, config, dtype, device)
    adapt = (lambda name, t: arch.adapt_tensor(config, name, t)) if arch.adapt_tensor else None
    tensors = load_checkpoint(model_dir, model.weight_specs(), dtype, device, adapt, arch.ignore_tensor)
    model.load_weights(tensors)
    return arch, config, model
