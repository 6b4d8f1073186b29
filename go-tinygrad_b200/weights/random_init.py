"""Random-weights mode: write a model folder from a configuration and a seed.

The folder holds ``config.json`` and ``model.safetensors`` and is read back
like any checkpoint.  Which tensors exist, and their shapes, come from the
architecture's plan, not from this file.  Each tensor's values depend on
(seed, tensor name) only, so adding a tensor does not change the others.
The reference has no such mode; its tests build tiny models by hand
(model/llama_test.go:180-198).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Mapping, Optional

import torch

from ..config.registry import find_architecture
from .binder import check_specs
from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensors(specs, seed: int, std: Optional[float], norm_std: float,
                   store_dtype: torch.dtype, device: str = "cpu") -> Mapping[str, torch.Tensor]:
    """Random values for every required spec.  Drawn on `device`: the host's and
    a GPU's generators give different (equally valid) values for one seed."""
    out = {}
    for s in check_specs(specs):
        if s.optional:
            continue
        g = torch.Generator(device=device)
        g.manual_seed(_tensor_seed(seed, s.name))
        scale = norm_std if s.role == "vector" else (s.std if std is None else std)
        t = torch.randn(s.shape, generator=g, dtype=torch.float32, device=device)
        out[s.name] = (s.mean + scale * t).to(store_dtype)
    return out


def write_random_model(folder: str, config_json: Mapping, seed: int = 0, *,
                       dtype: str = "bfloat16", std: Optional[float] = None,
                       norm_std: float = 0.0) -> str:
    """Create `folder` with config.json and model.safetensors.

    `config_json` is the architecture's config.json content (a dict, or a typed
    configuration with ``to_json()``).  Matrices and tables are N(0, std)
    (each spec's own default when `std` is None), norm scales 1 + N(0, norm_std).
    `dtype` is the storage dtype of every tensor.
    """
    from ..parts.plan import plan_weight_specs  # late: parts import weights
    if hasattr(config_json, "to_json"):
        config_json = config_json.to_json()
    if dtype not in _STORE:
        raise ValueError(f"dtype must be one of {sorted(_STORE)}, got {dtype!r}")
    arch = find_architecture(config_json)
    config = arch.read_config(config_json)
    plan = arch.plan(config)
    tensors = random_tensors(plan_weight_specs(plan), seed, std, norm_std, _STORE[dtype])
    os.makedirs(folder, exist_ok=True)
    raw = dict(config_json)
    raw["torch_dtype"] = dtype
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return folder
