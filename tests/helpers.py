"""Shared by the tests: tiny model folders, plain-implementation logits, host-side runners."""
from __future__ import annotations

import os

import torch
from safetensors.torch import load_file

import plain_gemma as plain
from tiny_configs import CONFIGS, SEEDS


def make_folder(tmp_path, name: str, dtype=torch.bfloat16) -> str:
    from wllm_b200.weights import write_random_model
    folder = os.path.join(str(tmp_path), f"tiny_{name}")
    write_random_model(folder, CONFIGS[name], SEEDS[name], dtype=dtype)
    return folder


def folder_weights(folder: str) -> dict:
    return {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


def random_requests(name: str, lengths, seed: int) -> dict:
    g = torch.Generator().manual_seed(seed)
    vocab = CONFIGS[name]["vocab_size"]
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lengths)}


def plain_rows(folder: str, name: str, requests: dict) -> dict:
    """{(request id, position): logits row} from the plain implementation, whole sequences."""
    w = folder_weights(folder)
    rows = {}
    for rid, toks in requests.items():
        logits = plain.forward(toks, w, CONFIGS[name])
        for p in range(len(toks)):
            rows[(rid, p)] = logits[p]
    return rows


class HostRing:
    """Stands in for the engine's ring of pinned staging buffers when a runner is put on the CPU for a test:
    the index arrays go to their place with a plain copy."""

    def send(self, host, dst) -> None:
        dst[:host.shape[0]].copy_(torch.from_numpy(host))


def host_runner(folder: str, dtype, page_size: int, num_pages: int, max_requests: int = 8):
    """A runner on the CPU for host-logic tests; the kernels must be replaced by
    kernel_refs.install(monkeypatch) first, and the staging ring by a plain copy."""
    from wllm_b200.cache import CacheManager
    from wllm_b200.config import config_from_folder
    from wllm_b200.engine import ComposedModel, ModelRunner
    from wllm_b200.weights import load_weights
    arch, cfg = config_from_folder(folder)
    model = ComposedModel(arch.make_plan(cfg), dtype)
    load_weights(model, folder, "cpu")
    cache = CacheManager(model.group_specs, page_size, num_pages, max_requests, model.state_specs, dtype, "cpu")
    runner = ModelRunner(model, cache, "cpu")
    runner._ring = HostRing()
    return runner


def max_diff(rows: dict, ref: dict) -> float:
    assert set(rows) == set(ref), f"{len(set(ref) - set(rows))} rows missing, {len(set(rows) - set(ref))} extra"
    return max(float((rows[k].double() - ref[k].double()).abs().max()) for k in ref)
