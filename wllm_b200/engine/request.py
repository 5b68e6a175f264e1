"""A request on its way through the engine."""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

from ..sampling.params import SamplingParams


class RequestStatus(Enum):
    WAITING = "waiting"          # queued (new, or preempted and waiting to be run again)
    PREFILLING = "prefilling"    # admitted; part of its known tokens is not in the cache yet
    RUNNING = "running"          # all but its newest token are in the cache: it decodes
    FINISHED = "finished"


@dataclass
class Request:
    """States and finishing rule follow the reference's Sequence (src/wllm/engine/sequence.py:13-59):
    a request ends on its end-of-sequence id (kept in the output), on a stop id, or at max_tokens."""
    request_id: object
    prompt_token_ids: list
    sampling: SamplingParams = field(default_factory=SamplingParams)
    eos_token_id: int | None = None
    output_token_ids: list = field(default_factory=list)
    logprobs: list = field(default_factory=list)
    status: RequestStatus = RequestStatus.WAITING
    finish_reason: str | None = None
    seed: int = 0                 # resolved at admission: sampling.seed, or drawn by the engine
    cache: object = None          # RequestCache while admitted
    num_computed: int = 0         # tokens whose keys and values are in the cache
    preemptions: int = 0
    seen: set = field(default_factory=set)   # distinct generated ids, for the repetition penalty
    inflight: int = 0             # 1 while its newest token is sampled on the device and not yet read
    inflight_row: int = -1        # that token's row among the sampled tokens of the step before

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    def token_at(self, i: int) -> int:
        n = len(self.prompt_token_ids)
        return self.prompt_token_ids[i] if i < n else self.output_token_ids[i - n]

    def tokens(self, start: int, stop: int) -> list:
        n = len(self.prompt_token_ids)
        if stop <= n:
            return self.prompt_token_ids[start:stop]
        return [self.token_at(i) for i in range(start, stop)]

    @property
    def worst_case_tokens(self) -> int:
        return len(self.prompt_token_ids) + self.sampling.max_tokens

    def append_token(self, token: int, logprob: float, max_model_len: int) -> None:
        self.output_token_ids.append(token)
        self.logprobs.append(logprob)
        self.seen.add(token)
        sp = self.sampling
        if (self.eos_token_id is not None and token == self.eos_token_id and not sp.ignore_eos) \
                or token in sp.stop_token_ids:
            self.status, self.finish_reason = RequestStatus.FINISHED, "stop"
        elif len(self.output_token_ids) >= sp.max_tokens or self.num_tokens >= max_model_len:
            self.status, self.finish_reason = RequestStatus.FINISHED, "length"

    @property
    def finished(self) -> bool:
        return self.status == RequestStatus.FINISHED
