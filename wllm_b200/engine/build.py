"""From a model folder (or a configuration and a seed) to a runner that can step."""
from __future__ import annotations

import torch

from ..cache import CacheManager
from ..config import EngineConfig, config_from_folder, resolve_architecture
from ..kernels.build import KernelBuildError
from ..weights import fill_random, load_weights
from .model import ComposedModel
from .runner import ModelRunner


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise KernelBuildError(f"device {device}: the engine runs on a CUDA device only (sm_100a kernels, "
                               f"no CPU path); torch.cuda.is_available() = {torch.cuda.is_available()}")
    return device


def build_model(folder: str | None, dtype, device, config=None, random_seed: int | None = None) -> ComposedModel:
    """The loaded model of a folder; or, with `config` and `random_seed`, one with random weights."""
    device = require_cuda(device)
    if folder is not None:
        arch, cfg = config_from_folder(folder)
    else:
        if config is None or random_seed is None:
            raise ValueError("give a model folder, or a configuration and a seed for random weights")
        arch = resolve_architecture(config.architecture)
        cfg = config
    model = ComposedModel(arch.make_plan(cfg), dtype)
    model.config = cfg
    with torch.cuda.device(device):
        if folder is not None:
            load_weights(model, folder, device)
        else:
            fill_random(model, random_seed, device)
    return model


def build_runner(model: ComposedModel, engine: EngineConfig, num_pages: int | None = None,
                 poison_pages: bool = False) -> ModelRunner:
    device = require_cuda(engine.device)
    cache = CacheManager(model.group_specs, page_size=engine.block_size,
                         num_pages=num_pages if num_pages is not None else engine.num_blocks,
                         max_requests=engine.max_num_seqs, states=model.state_specs, dtype=model.dtype, device=device,
                         poison=poison_pages)
    return ModelRunner(model, cache, device)
