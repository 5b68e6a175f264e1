"""The Python entry point: token ids in, generated token ids out.

    llm = LLM("/path/to/model", dtype="bfloat16", num_blocks=4096, chunked_prefill_tokens=2048)
    outs = llm.generate([[2, 651, 6037]], SamplingParams(temperature=0.8, seed=1, max_tokens=32))

The reference has no single class for offline use; it is assembled by hand from
load_native, KVCacheManager, Scheduler, add_request and run_to_completion
(tests/test_gemma_architecture.py:119-124).  `LLM` wraps that assembly, with the
reference's option names: num_blocks, block_size, dtype, chunked_prefill_tokens,
cuda_graphs (src/wllm/cli.py:30-35).  `add_request` / `step` expose the loop itself.
"""
from __future__ import annotations

from dataclasses import dataclass

from .config import EngineConfig
from .engine.build import build_model, build_runner
from .engine.request import Request
from .engine.scheduler import Scheduler
from .sampling import SamplingParams
from .sampling.sampler import Sampler


@dataclass
class RequestOutput:
    request_id: object
    prompt_token_ids: list
    token_ids: list
    logprobs: list
    finish_reason: str | None
    preemptions: int = 0


class LLM:
    def __init__(self, model: str | None = None, *, config=None, random_seed: int | None = None,
                 dtype="bfloat16", block_size: int = 16, num_blocks: int = 256,
                 chunked_prefill_tokens: int | None = None, max_num_seqs: int = 256, max_model_len: int | None = None,
                 cuda_graphs: bool = False, device: str = "cuda:0", admission: str = "worst_case", seed: int = 0,
                 async_scheduling: bool = False, poison_pages: bool = False, prefill_row_quantum: int | None = None):
        """`model`: a folder with config.json and model.safetensors.  Without it, `config` (a typed
        configuration) and `random_seed` make a model with random weights on the device."""
        self.engine_config = EngineConfig(dtype=dtype, block_size=block_size, num_blocks=num_blocks,
                                          chunked_prefill_tokens=chunked_prefill_tokens, max_num_seqs=max_num_seqs,
                                          max_model_len=max_model_len, cuda_graphs=cuda_graphs, device=device,
                                          poison_pages=poison_pages, prefill_row_quantum=prefill_row_quantum)
        ec = self.engine_config
        self.model = build_model(model, ec.dtype, ec.device, config=config, random_seed=random_seed)
        self.runner = build_runner(self.model, ec, poison_pages=ec.poison_pages)
        if cuda_graphs:
            self.runner.enable_graphs()
        self.sampler = Sampler(ec.device)
        self.scheduler = Scheduler(self.runner, self.sampler, chunked_prefill_tokens=chunked_prefill_tokens,
                                   max_num_seqs=max_num_seqs, max_model_len=max_model_len, admission=admission, seed=seed,
                                   async_scheduling=async_scheduling, row_quantum=ec.prefill_row_quantum)
        self.eos_token_id = self.model.plan.eos_token_id
        self._next_id = 0

    def add_request(self, prompt_token_ids, sampling_params: SamplingParams | None = None, request_id=None) -> Request:
        if request_id is None:
            request_id = self._next_id
            self._next_id += 1
        req = Request(request_id, list(prompt_token_ids), sampling_params or SamplingParams(),
                      eos_token_id=self.eos_token_id)
        self.scheduler.add_request(req)
        return req

    def step(self) -> list:
        """One scheduler step; returns the requests that got a token (with `async_scheduling`: the tokens of
        the step before, read while this one runs)."""
        return self.scheduler.step()

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    def generate(self, prompts, sampling_params=None) -> list:
        """Generate for a batch of prompts (lists of token ids); results in the order of the prompts."""
        prompts = [list(p) for p in prompts]
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams for all prompts, or one per prompt")
        reqs = [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        self.scheduler.run_to_completion()
        return [RequestOutput(r.request_id, r.prompt_token_ids, list(r.output_token_ids), list(r.logprobs),
                              r.finish_reason, r.preemptions) for r in reqs]

    @property
    def stats(self) -> dict:
        s = dict(self.scheduler.stats)
        s["pages_high_water"] = list(self.runner.cache.pages_high_water)
        return s
