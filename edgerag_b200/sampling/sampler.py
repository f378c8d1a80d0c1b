"""Sampling above the step function: float32 logits rows in, one token id per row out.

One kernel launch covers all rows of a step (greedy rows and temperature rows together) and one
small device-to-host copy brings the ids back; the reference does an ``int(argmax)`` per request
(edgerag/serve/executor.py:136,154).  Launching and reading are separate, so that the engine can
launch the next step while the ids of this one are still on their way.
"""

from __future__ import annotations

import numpy as np
import torch

from ..ops import kernels
from .params import SamplingParams, as_int64, rng_state


class PendingTokens:
    """Tokens of one ``launch`` that are on their way to the host."""

    def __init__(self, n: int, host: torch.Tensor, event: torch.cuda.Event) -> None:
        self.n, self._host, self._event = n, host, event

    def read(self) -> list[int]:
        """Wait for the copy and return the ids (may be called once per launch, in launch order)."""
        self._event.synchronize()
        return self._host[: self.n].tolist()


class Sampler:
    """``launch`` enqueues the kernel and the copy to the host and returns at once; ``read`` on what
    it returns waits for them.  Up to ``RING`` launches may be outstanding.  ``device_tokens`` holds
    the ids of the latest launch on the device, row by row, for a next step that is launched before
    the host has read them."""

    RING = 4

    def __init__(self, device: torch.device, max_rows: int = 256) -> None:
        self.device = device
        self._turn = 0
        self._grow(max_rows)

    def _grow(self, rows: int) -> None:
        self.max_rows = rows
        self._tokens = torch.empty(rows, dtype=torch.int32, device=self.device)
        self._temps = torch.empty(rows, dtype=torch.float32, device=self.device)
        self._states = torch.empty(rows, dtype=torch.int64, device=self.device)
        self._host_tokens = [torch.empty(rows, dtype=torch.int32, pin_memory=True) for _ in range(self.RING)]
        self._host_temps = [torch.empty(rows, dtype=torch.float32, pin_memory=True) for _ in range(self.RING)]
        self._host_states = [torch.empty(rows, dtype=torch.int64, pin_memory=True) for _ in range(self.RING)]
        self._events = [torch.cuda.Event() for _ in range(self.RING)]
        self._used = [False] * self.RING

    @property
    def device_tokens(self) -> torch.Tensor:
        return self._tokens

    def launch(self, logits: torch.Tensor, params: list[SamplingParams], seeds: list[int],
               token_indices: list[int]) -> PendingTokens:
        """``params[r]``, ``seeds[r]`` and ``token_indices[r]`` belong to row ``r`` of ``logits``."""
        n = logits.shape[0]
        if not (len(params) == len(seeds) == len(token_indices) == n):
            raise ValueError("one SamplingParams, seed and token index per logits row")
        if n > self.max_rows:
            torch.cuda.current_stream().synchronize()     # nothing may still point at the old buffers
            self._grow(2 * n)
        i = self._turn = (self._turn + 1) % self.RING
        if self._used[i]:
            self._events[i].synchronize()                  # the staging buffers of this turn are free again
        if all(p.greedy for p in params):
            kernels.sample_rows(logits, self._tokens[:n])
        else:
            self._host_temps[i][:n].copy_(torch.from_numpy(np.asarray([p.temperature for p in params], dtype=np.float32)))
            self._host_states[i][:n].copy_(torch.from_numpy(
                np.asarray([as_int64(rng_state(s, k)) for s, k in zip(seeds, token_indices)], dtype=np.int64)))
            self._temps[:n].copy_(self._host_temps[i][:n], non_blocking=True)
            self._states[:n].copy_(self._host_states[i][:n], non_blocking=True)
            kernels.sample_rows(logits, self._tokens[:n], self._temps[:n], self._states[:n])
        self._host_tokens[i][:n].copy_(self._tokens[:n], non_blocking=True)
        self._events[i].record()
        self._used[i] = True
        return PendingTokens(n, self._host_tokens[i], self._events[i])

    def sample(self, logits: torch.Tensor, params: list[SamplingParams], seeds: list[int],
               token_indices: list[int]) -> list[int]:
        return self.launch(logits, params, seeds, token_indices).read()
