"""A request as the engine tracks it (the reference's ``Sequence``,
turingserve/engine/sequence.py:18-56): its tokens so far, how many are in the cache, its status."""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

from turingserve_b200.cache.manager import RequestCache
from turingserve_b200.sampling.params import SamplingParams


class Status(Enum):
    WAITING = 0
    RUNNING = 1
    FINISHED = 2


@dataclass
class Request:
    request_id: str
    token_ids: list[int]                 # prompt, then generated tokens
    num_prompt_tokens: int
    params: SamplingParams
    seed: int = 0
    cache: RequestCache | None = None    # None while waiting (or after preemption)
    status: Status = Status.WAITING
    finish_reason: str | None = None
    num_drawn: int = 0                   # tokens sampled so far = position in its random stream
    pending: bool = False                # the last entry of token_ids is a stand-in for a token in flight
    num_preemptions: int = 0

    @property
    def num_computed(self) -> int:
        return 0 if self.cache is None else self.cache.num_tokens

    @property
    def num_uncomputed(self) -> int:
        return len(self.token_ids) - self.num_computed

    @property
    def num_output(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def output_ids(self) -> list[int]:
        return self.token_ids[self.num_prompt_tokens:]

    @property
    def finished(self) -> bool:
        return self.status == Status.FINISHED


@dataclass
class Scheduled:
    request: Request
    num_tokens: int
    samples: bool                        # the portion reaches the end of token_ids


@dataclass
class BatchPlan:
    items: list[Scheduled] = field(default_factory=list)
    num_decode: int = 0
    num_tokens: int = 0
    preempted: list[Request] = field(default_factory=list)
    failed: list[Request] = field(default_factory=list)      # can never fit: to be finished with "error"


@dataclass
class RequestOutput:
    request_id: str
    delta_token_ids: list[int]
    finished: bool
    finish_reason: str | None
    prompt_tokens: int
    completion_tokens: int
