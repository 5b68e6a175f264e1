"""The plan of a model: its blocks (specs) and the order in which they run (data).

`runs` is a list: entry i runs block `block` with a cache of its own, or, with
`cache_from = j`, reads the cache that run j writes (and writes none).  A block may
appear in several runs (shared weights); each such run has its own cache unless it
names another's.  An architecture is added by a function from its configuration to
a `ModelPlan`; the engine builds the same `ComposedModel` from any plan.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import PartSpec


@dataclass(frozen=True)
class LayerRun:
    block: int
    cache_from: int | None = None


@dataclass
class ModelPlan:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    blocks: list
    final_norm: PartSpec
    head: PartSpec
    runs: list = field(default_factory=list)
    eos_token_id: int | None = None
    bos_token_id: int | None = None

    def __post_init__(self):
        if not self.runs:
            self.runs = [LayerRun(i) for i in range(len(self.blocks))]
        for i, r in enumerate(self.runs):
            if not 0 <= r.block < len(self.blocks):
                raise ValueError(f"run {i} names block {r.block}, but there are {len(self.blocks)} blocks")
            if r.cache_from is not None and not (0 <= r.cache_from < i and self.runs[r.cache_from].cache_from is None):
                raise ValueError(f"run {i} reads the cache of run {r.cache_from}, which must be an earlier run "
                                 f"with a cache of its own")
