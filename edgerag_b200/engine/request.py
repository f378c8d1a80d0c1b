"""A generation request and its life cycle (tensor-free apart from carrying ``prompt_embeds``).

States and fields follow the reference's ``Request`` (edgerag/sched/request.py:23-172): WAITING ->
PREFILLING -> DECODING -> FINISHED, plus REJECTED; ``prefill_offset`` became ``num_computed``, the
number of tokens of ``prompt + generated`` whose keys and values are in the cache.  A request is
"prefilling" while more than one token is still to be fed and "decoding" when exactly one is, so
a request that was preempted and recomputes its prompt and its generated tokens needs no special
path: it is simply prefilling again.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Any

from ..sampling.params import SamplingParams


class RequestState(str, Enum):
    WAITING = "waiting"
    PREFILLING = "prefilling"
    DECODING = "decoding"
    FINISHED = "finished"
    REJECTED = "rejected"


@dataclass
class Request:
    request_id: str
    prompt_token_ids: list[int]
    sampling: SamplingParams = field(default_factory=SamplingParams)
    #: ``[prompt_len, hidden]`` rows that replace the embedding lookup for the prompt
    #: (edgerag/sched/request.py:58-69); ``prompt_token_ids`` then only carries the length.
    prompt_embeds: Any = None
    seed: int = 0
    state: RequestState = RequestState.WAITING
    num_computed: int = 0
    generated_token_ids: list[int] = field(default_factory=list)
    arrival_step: int = 0
    admitted_step: int | None = None
    first_token_step: int | None = None
    finished_step: int | None = None
    preemptions: int = 0
    finish_reason: str | None = None

    @property
    def prompt_len(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def max_new_tokens(self) -> int:
        return self.sampling.max_new_tokens

    @property
    def num_generated(self) -> int:
        return len(self.generated_token_ids)

    @property
    def total_tokens(self) -> int:
        return self.prompt_len + self.num_generated

    @property
    def final_tokens(self) -> int:
        """Positions the request occupies when it has generated everything it may."""
        return self.prompt_len + self.max_new_tokens

    @property
    def pending(self) -> int:
        """Tokens of ``prompt + generated`` not yet in the cache."""
        return self.total_tokens - self.num_computed

    @property
    def is_finished(self) -> bool:
        return self.state in (RequestState.FINISHED, RequestState.REJECTED)

    def next_portion(self, limit: int) -> tuple[int, int, bool]:
        """``(start, n, from_embeds)`` of the next tokens to feed, at most ``limit`` of them.

        A portion never crosses from the embedded prompt into generated ids, so an entry of a
        step carries either embedding rows or token ids.
        """
        if limit <= 0:
            raise ValueError(f"portion limit must be positive, got {limit}")
        start = self.num_computed
        n = min(limit, self.pending)
        from_embeds = self.prompt_embeds is not None and start < self.prompt_len
        if from_embeds:
            n = min(n, self.prompt_len - start)
        return start, n, from_embeds

    def token_at(self, i: int) -> int:
        return self.prompt_token_ids[i] if i < self.prompt_len else self.generated_token_ids[i - self.prompt_len]

    def should_stop(self, eos_token_id: int | None) -> bool:
        """edgerag/sched/request.py:126-133."""
        if self.num_generated >= self.max_new_tokens:
            return True
        return bool(eos_token_id is not None and self.generated_token_ids
                    and self.generated_token_ids[-1] == eos_token_id)

    def to_dict(self) -> dict[str, Any]:
        return {
            "request_id": self.request_id, "state": self.state.value, "prompt_len": self.prompt_len,
            "num_computed": self.num_computed, "generated": self.num_generated,
            "preemptions": self.preemptions, "finish_reason": self.finish_reason,
            "arrival_step": self.arrival_step, "first_token_step": self.first_token_step,
            "finished_step": self.finished_step,
        }
