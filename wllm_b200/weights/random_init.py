"""Random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed, or the same distributions made directly on the device.

Matrices and tables are N(0, std), vectors (norm gains) N(0, vector_std); tensors
are drawn one by one from one seeded CPU generator in the order the model lists
them, so the folder is reproducible bit for bit.  The reference has no such mode:
its tests lean on torch's default initialisation under a manual seed
(tests/test_cpu_inference.py:30-39).
"""
from __future__ import annotations

import json
import os

import torch
from safetensors.torch import save_file

from ..config.registry import resolve_architecture


def _typed(config):
    """(architecture entry, typed configuration) from a typed configuration or a raw dictionary."""
    if isinstance(config, dict):
        arch = resolve_architecture(config.get("architectures") or [])
        return arch, arch.config_class.from_dict(config, where="configuration")
    return resolve_architecture(config.architecture), config


def random_tensors(config, seed: int, dtype=torch.bfloat16, std: float = 0.02, vector_std: float = 0.1) -> dict:
    from ..engine.model import ComposedModel
    arch, cfg = _typed(config)
    model = ComposedModel(arch.make_plan(cfg), dtype)
    g = torch.Generator().manual_seed(seed)
    out = {}
    for ps in model.param_specs():
        s = vector_std if ps.kind == "vector" else std
        out[ps.name] = (torch.randn(tuple(ps.shape), generator=g, dtype=torch.float32) * s).to(dtype)
    return out


def write_random_model(folder: str, config, seed: int, dtype=torch.bfloat16, std: float = 0.02,
                       vector_std: float = 0.1) -> str:
    """Write `folder/config.json` and `folder/model.safetensors`; returns the folder."""
    _, cfg = _typed(config)
    os.makedirs(folder, exist_ok=True)
    raw = cfg.to_dict()
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}[dtype]
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(raw, f, indent=1)
    save_file(random_tensors(cfg, seed, dtype, std, vector_std), os.path.join(folder, "model.safetensors"))
    return folder


def fill_random(model, seed: int, device, std: float = 0.02, vector_std: float = 0.1) -> None:
    """Fill a ComposedModel with random weights made on the device (no folder, no host copy)."""
    g = torch.Generator(device=device).manual_seed(seed)
    kinds = {ps.name: ps for ps in model.param_specs()}

    def fetch(name: str) -> torch.Tensor:
        ps = kinds[name]
        s = vector_std if ps.kind == "vector" else std
        t = torch.randn(tuple(ps.shape), generator=g, dtype=torch.float32, device=device) * s
        return t.to(model.dtype)
    model.load(fetch)
