"""Random weights for a configuration: as a model folder on disk (config.json and
model.safetensors), or as tensors made on the device for models too large to be
worth a file.  The reference has no such mode; its tests download checkpoints
(tests/test_model_generation.py:94-111).

A tensor's values depend on the seed and on the tensor's name only, so the same
seed gives the same folder whatever the order of tensors.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict, Mapping, Optional

import torch

from ..parts.base import WeightSpec
from .safetensors_io import save_file


def _generator(seed: int, name: str, device: "torch.device | str" = "cpu") -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode("utf-8"))) & 0x7FFFFFFFFFFFFFFF)
    return g


def random_tensors(specs: Mapping[str, WeightSpec], seed: int, dtype: torch.dtype = torch.bfloat16,
                   std: float = 0.02, norm_mean: float = 1.0, device: "torch.device | str" = "cpu",
                   ) -> Dict[str, torch.Tensor]:
    """Matrices ~ N(0, std); vectors (norm weights) ~ norm_mean + N(0, std)."""
    out: Dict[str, torch.Tensor] = {}
    for name, spec in specs.items():
        g = _generator(seed, name, device)
        if spec.role == "table":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
            continue
        t = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device) * std
        if spec.role == "vector":
            t += norm_mean
        out[name] = t.to(dtype)
    return out


def write_model_folder(config, specs: Mapping[str, WeightSpec], out_dir: str, seed: int,
                       dtype: torch.dtype = torch.bfloat16, std: float = 0.02, norm_mean: float = 1.0) -> str:
    """Writes config.json and model.safetensors for ``config`` (a typed configuration
    with ``to_dict``) and returns the folder."""
    os.makedirs(out_dir, exist_ok=True)
    data = config.to_dict()
    data["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(data, f, indent=2)
    tensors = random_tensors(specs, seed, dtype, std, norm_mean)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"),
              metadata={"format": "pt", "seed": str(seed), "std": str(std)})
    return out_dir
