"""Engine options: the knobs of cache, batching and precision.

Names follow the reference's command line where it has them
(src/wllm/cli.py:30-35: --num-blocks, --block-size, --dtype,
--chunked-prefill-tokens); the rest are this engine's own.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .base import ConfigError

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ConfigError(f"dtype {name}: the engine runs bfloat16 or float32")
        return name
    if name not in DTYPES:
        raise ConfigError(f"dtype {name!r}: choose bfloat16 or float32")
    return DTYPES[name]


@dataclass
class EngineConfig:
    dtype: torch.dtype = torch.bfloat16
    block_size: int = 16                 # tokens per cache page
    num_blocks: int = 256                # pages in each cache group's pool
    chunked_prefill_tokens: int | None = None   # token budget of one step; None = whole prompts
    prefill_row_quantum: int | None = None     # rows of a tile of the products of a step of many rows (scheduler: 'rows');
                                               # None: 256 under bfloat16 (pairs of CTAs), off under float32
    max_num_seqs: int = 256              # requests that may be live at once (table rows, state slots)
    max_model_len: int | None = None     # None: the model's max_position_embeddings
    cuda_graphs: bool = False            # replay captured graphs for decode-only steps
    device: str = "cuda:0"
    poison_pages: bool = False           # debugging: cache pages hold NaN until written and again once given back

    def __post_init__(self):
        self.dtype = parse_dtype(self.dtype)
        if self.block_size < 16 or self.block_size & (self.block_size - 1):
            raise ConfigError(f"block_size {self.block_size}: a page holds a power of two of at least 16 tokens")
        if self.num_blocks < 1:
            raise ConfigError("num_blocks must be at least 1")
        if self.chunked_prefill_tokens is not None and self.chunked_prefill_tokens < 1:
            raise ConfigError("chunked_prefill_tokens must be at least 1 (or None for whole prompts)")
        if self.prefill_row_quantum is None:
            self.prefill_row_quantum = 256 if self.dtype == torch.bfloat16 else 0
        if self.prefill_row_quantum < 0:
            raise ConfigError("prefill_row_quantum must be 0 (off) or a number of rows")
        if self.max_num_seqs < 1:
            raise ConfigError("max_num_seqs must be at least 1")
