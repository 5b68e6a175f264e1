"""What a model is put together from: specs (data), parts (code), registries (names).

A *spec* says which part stands at a place and with which sizes and constants; it is
plain data made from the configuration, layer by layer.  A *part* is the code for one
kind of spec.  No part knows which model it is in: it gets its sizes, constants and
the checkpoint names of its tensors from its spec, and the step's batch from the
`StepContext`.  Five registries map a spec's `kind` to the class that runs it:

    NORMS          x (and a pending branch output) -> normed x
    POSITIONS      how a mixer encodes positions
    MIXERS         the part that mixes tokens (attention here); may need cache or state
    FEED_FORWARDS  the per-token part (dense, gated, experts)
    BLOCKS         how norms, mixer and feed-forward are arranged around the residual

Interfaces (duck-typed; see the built-in parts for examples):

    every part      __init__(spec, hidden_size, model_dtype), param_specs() -> [ParamSpec],
                    load(fetch) where fetch(name) returns the checkpoint tensor on the device
    norm            __call__(residual: Residual, ctx) -> tensor [n, hidden] in the model dtype
                    rows(residual, rows, ctx) -> the same at selected rows only
    position        an object the mixer of its kind understands (rotary: .inv_freq, .rotary_dim, and
                    optionally .pairing = 'half' | 'interleaved')
    mixer           cache_need() -> KVNeed | StateNeed | None
                    __call__(x, ctx, cache: CacheRef) -> tensor [n, hidden]
    feed-forward    __call__(x, ctx) -> tensor [n, hidden]
    block           __call__(residual, ctx, cache: CacheRef) -> None (updates the residual)
    embedding       __call__(token_ids, ctx) -> float32 tensor [n, hidden] (the residual stream)
    head            __init__(..., embedding) gets the model's embedding part (for a tied table);
                    __call__(hidden_rows, ctx) -> float32 logits [rows, vocab]

A part may declare `graph_safe = True`: everything it launches depends on device data and on the step's
size bounds alone (tokens, requests, table width, longest context rounded to the table's reach), never on
host copies of the batch's contents, and running the same step twice leaves the same cache and state.  Decode
steps are replayed from captured CUDA graphs only for models whose parts all say so and that declare no
per-request state; any other model runs every step eagerly, whatever `cuda_graphs` asks for.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch


@dataclass(frozen=True)
class ParamSpec:
    """One checkpoint tensor a part reads.  kind: 'matrix' and 'table' are held in the
    model's element type; 'vector' (norm gains and the like) keeps a 32-bit storage type."""
    name: str
    shape: tuple
    kind: str = "matrix"


@dataclass(frozen=True)
class PartSpec:
    kind: str
    options: dict = field(default_factory=dict)

    def __getattr__(self, key: str) -> Any:
        try:
            return self.__dict__["options"][key]
        except KeyError:
            raise AttributeError(f"{self.kind} spec has no option '{key}'") from None


def spec(kind: str, **options) -> PartSpec:
    return PartSpec(kind, options)


@dataclass(frozen=True)
class KVNeed:
    """A mixer that reads keys and values from pages."""
    kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps per-request state of fixed size: name -> (shape, dtype)."""
    tensors: tuple   # of (name, shape, dtype)


@dataclass
class CacheRef:
    """Where a layer run finds its cache: pages of (group, layer), or state tensors by name.
    `writes` is false for a run that reads another run's cache."""
    group: int | None = None
    layer: int | None = None
    writes: bool = True
    state_names: dict | None = None   # mixer's own name -> name in the manager's state slots


class Partials:
    """A branch output still in parts: [parts, n, hidden] float32 partial sums (a split-K product), which the
    next norm adds in order while it folds them into the residual."""

    def __init__(self, tensor: torch.Tensor):
        self.tensor, self.parts = tensor, tensor.shape[0]


def as_branch(product):
    """What ops.project returned, as a branch output: a tensor, or Partials."""
    tensor, parts = product
    return Partials(tensor) if parts else tensor


class Residual:
    """The residual stream in 32-bit, and the branch output not yet added to it (a tensor [n, hidden], or
    `Partials`).  The next norm folds `pending` in (one kernel), so no separate add is launched."""

    def __init__(self, stream: torch.Tensor):
        self.stream = stream
        self.pending = None

    def pending_args(self) -> tuple:
        """(delta tensor or None, number of parts) for the norm kernel."""
        if isinstance(self.pending, Partials):
            return self.pending.tensor, self.pending.parts
        return self.pending, 0


class Registry(dict):
    def __init__(self, what: str):
        super().__init__()
        self.what = what

    def register(self, kind: str):
        def wrap(cls):
            self[kind] = cls
            return cls
        return wrap

    def build(self, part_spec: PartSpec, **kwargs):
        if part_spec.kind not in self:
            raise KeyError(f"no {self.what} of kind '{part_spec.kind}' is registered (known: {', '.join(sorted(self))})")
        return self[part_spec.kind](part_spec, **kwargs)


EMBEDDINGS = Registry("embedding")
HEADS = Registry("logits head")
NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block arrangement")
