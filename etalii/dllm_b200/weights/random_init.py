"""The random-weights mode: writes a model folder (config.json, model.safetensors) from a configuration and a seed.

Every tensor has a random stream of its own, keyed by (seed, tensor name), so the numbers do not depend on the
order or on which other tensors exist. Matrices are N(0, std); norm weights 1 + N(0, std / 2). Values are drawn in
float32 on the CPU and stored in `dtype` (bfloat16 by default, as checkpoints of this family are).
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

from ..config.registry import architecture
from .loader import expected_tensors
from .safetensors_io import write_safetensors


def _stream(seed: int, name: str) -> torch.Generator:
    digest = hashlib.sha256(f"{int(seed)}:{name}".encode("utf-8")).digest()
    generator = torch.Generator(device="cpu")
    generator.manual_seed(int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF)
    return generator


def random_tensors(config, seed: int, dtype: torch.dtype = torch.bfloat16, std: float = 0.02) -> dict:
    spec = architecture(config.model_type).build_spec(config)
    out = {}
    for name, param in expected_tensors(spec).items():
        generator = _stream(seed, name)
        if param.init == "int":
            out[name] = torch.randint(0, 2**15, tuple(param.shape), generator=generator, dtype=torch.int32)
            continue
        values = torch.randn(tuple(param.shape), generator=generator, dtype=torch.float32)
        if param.init == "ones":
            values = 1.0 + values * (std / 2)
        else:
            values = values * std
        out[name] = values.to(dtype)
    return out


def write_random_model(folder: str, config, seed: int, dtype: torch.dtype = torch.bfloat16, std: float = 0.02) -> str:
    """Writes `folder/config.json` and `folder/model.safetensors`; returns the folder."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(config.to_hf(), handle, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), random_tensors(config, seed, dtype, std))
    return folder


def write_model(folder: str, config_dict: dict, tensors: dict) -> str:
    """Writes a model folder from a config.json dict and named tensors (used by tests and tools)."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(config_dict, handle, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder
