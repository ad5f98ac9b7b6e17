"""What the engine keeps per request, and what it hands back per step.

The reference tracks the same facts in its ``Sequence`` (turingserve/engine/sequence.py:18-56):
the tokens so far (prompt, then generated), how many of them are in the cache, and where the
request stands.  Here the cache manager owns the count of cached tokens (``RequestCache``), so a
request without a ``cache`` is by construction one that holds no pages: queued, or preempted and
queued again.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum

from turingserve_b200.cache.manager import RequestCache
from turingserve_b200.sampling.params import SamplingParams


class Status(Enum):
    WAITING = "waiting"          # in the scheduler's queue, holding nothing
    RUNNING = "running"          # admitted: holds a state slot and pages
    FINISHED = "finished"


@dataclass
class Request:
    request_id: str
    token_ids: list[int]
    num_prompt_tokens: int
    params: SamplingParams
    seed: int = 0                          # of this request's random stream
    num_drawn: int = 0                     # position in that stream: tokens sampled so far
    cache: RequestCache | None = None
    status: Status = Status.WAITING
    finish_reason: str | None = None
    # True while the last entry of token_ids stands in for a token the GPU has not delivered yet
    pending: bool = False
    num_preemptions: int = 0

    # -- derived -------------------------------------------------------------------------------------
    @property
    def finished(self) -> bool:
        return self.status is Status.FINISHED

    @property
    def num_computed(self) -> int:
        """Tokens whose keys and values are in the cache."""
        return self.cache.num_tokens if self.cache is not None else 0

    @property
    def num_uncomputed(self) -> int:
        """Tokens still to run: 1 for a request that decodes, more in the middle of a prompt (or of
        a recompute after preemption)."""
        return len(self.token_ids) - self.num_computed

    @property
    def decoding(self) -> bool:
        return self.num_uncomputed == 1

    @property
    def output_ids(self) -> list[int]:
        return self.token_ids[self.num_prompt_tokens:]

    @property
    def num_output(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens


@dataclass
class RequestOutput:
    """One step's news about a request: the tokens it gained and, when it ended, why."""

    request_id: str
    delta_token_ids: list[int]
    finished: bool
    finish_reason: str | None
    prompt_tokens: int
    completion_tokens: int
