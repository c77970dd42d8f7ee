"""A request as the scheduler sees it (the reference's ``Sequence``:
``ginfer/engine/sequence.h:18-80``: token ids, state, prompt length, ``max_tokens``,
``ignore_eos``, three time stamps)."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field

from ..sampling.params import SamplingParams


class RequestState(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass
class Request:
    request_id: object
    prompt: list[int]
    params: SamplingParams
    seed: int = 0
    output: list[int] = field(default_factory=list)
    state: RequestState = RequestState.WAITING
    num_computed: int = 0            # tokens whose keys are in the cache
    finish_reason: str | None = None  # "eos" | "max_tokens" | "max_seq_len" | "out_of_pages"
    finish_pending: str | None = None  # ended, but still part of a step that is under way
    num_preemptions: int = 0
    arrival_time: float = 0.0
    first_token_time: float | None = None
    finish_time: float | None = None

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    def token_at(self, i: int) -> int:
        n = len(self.prompt)
        return self.prompt[i] if i < n else self.output[i - n]

    def tokens(self, start: int, stop: int) -> list[int]:
        n = len(self.prompt)
        if stop <= n:
            return self.prompt[start:stop]
        if start >= n:
            return self.output[start - n:stop - n]
        return self.prompt[start:] + self.output[:stop - n]
