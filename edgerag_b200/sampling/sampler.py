"""Sampling above the step function: float32 logits rows in, one token id per row out.

One kernel launch covers all rows of a step (greedy rows and temperature rows together) and one
small device-to-host copy brings the ids back; the reference does an ``int(argmax)`` per request
(edgerag/serve/executor.py:136,154).
"""

from __future__ import annotations

import numpy as np
import torch

from ..ops import kernels
from .params import SamplingParams, as_int64, rng_state


class Sampler:
    def __init__(self, device: torch.device, max_rows: int = 256) -> None:
        self.device = device
        self._grow(max_rows)

    def _grow(self, rows: int) -> None:
        self.max_rows = rows
        self._tokens = torch.empty(rows, dtype=torch.int32, device=self.device)
        self._temps = torch.empty(rows, dtype=torch.float32, device=self.device)
        self._states = torch.empty(rows, dtype=torch.int64, device=self.device)
        self._host_tokens = torch.empty(rows, dtype=torch.int32, pin_memory=True)

    def sample(self, logits: torch.Tensor, params: list[SamplingParams], seeds: list[int],
               token_indices: list[int]) -> list[int]:
        """``params[r]``, ``seeds[r]`` and ``token_indices[r]`` belong to row ``r`` of ``logits``."""
        n = logits.shape[0]
        if not (len(params) == len(seeds) == len(token_indices) == n):
            raise ValueError("one SamplingParams, seed and token index per logits row")
        if n > self.max_rows:
            self._grow(2 * n)
        if all(p.greedy for p in params):
            kernels.sample_rows(logits, self._tokens[:n])
        else:
            temps = np.asarray([p.temperature for p in params], dtype=np.float32)
            states = np.asarray([as_int64(rng_state(s, i)) for s, i in zip(seeds, token_indices)], dtype=np.int64)
            self._temps[:n].copy_(torch.from_numpy(temps))
            self._states[:n].copy_(torch.from_numpy(states))
            kernels.sample_rows(logits, self._tokens[:n], self._temps[:n], self._states[:n])
        self._host_tokens[:n].copy_(self._tokens[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._host_tokens[:n].tolist()
