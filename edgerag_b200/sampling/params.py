"""What a caller may ask of sampling.

The reference decodes greedily only and refuses anything else (edgerag/serve/app.py:105-120:
``temperature`` outside {None, 0} or ``top_p`` outside {None, 1} is an error).  Greedy is therefore
the default; temperature sampling with a seed is this engine's addition.  ``max_new_tokens``
defaults to 64 as in the reference's ``Request`` (edgerag/sched/request.py:50).
"""

from __future__ import annotations

from dataclasses import dataclass

_MASK = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int | None = None
    max_new_tokens: int = 64
    top_p: float | None = None

    def __post_init__(self) -> None:
        if self.temperature is None or self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.top_p not in (None, 1, 1.0):
            raise ValueError("top_p other than 1 is not supported (the reference refuses it too)")
        if self.max_new_tokens < 1:
            raise ValueError(f"max_new_tokens must be >= 1, got {self.max_new_tokens}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0


def rng_state(seed: int, token_index: int) -> int:
    """The 64-bit state from which the sampling kernel derives the uniform for one draw.

    A function of the request's seed and of the index of the token being generated only, so a
    request's draws do not depend on the batch it ran in, on how its prompt was cut, or on a
    preemption in between.
    """
    return (seed * 0x9E3779B97F4A7C15 + (token_index + 1) * 0xD1B54A32D192ED03 + 0x2545F4914F6CDD1D) & _MASK


def as_int64(state: int) -> int:
    """The same 64 bits as a signed value (what an int64 tensor holds)."""
    return state - (1 << 64) if state >= (1 << 63) else state
