"""The tensors behind the cache manager: page pools per group and state records per slot.

One allocation per cache group, made once (the reference's arena: edgerag/serve/executor.py:76-83),
laid out ``[layer, k|v, page, kv head, offset, head_dim]`` so that one (layer, page, head) is a
contiguous ``page_size * head_dim`` run: the unit an attention kernel streams.
"""

from __future__ import annotations

import torch

from .manager import CacheLayout

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class DevicePools:
    def __init__(self, layout: CacheLayout, page_size: int, num_pages: list[int], max_requests: int,
                 dtype: torch.dtype, device: torch.device, poison: bool = False) -> None:
        self.layout = layout
        self.page_size = page_size
        self.dtype = dtype
        self.device = device
        self.poison = poison
        self.kv: list[torch.Tensor] = []
        for g, n in zip(layout.groups, num_pages):
            shape = (g.n_layers, 2, n, g.n_kv_heads, page_size, g.head_dim)
            pool = torch.empty(shape, dtype=dtype, device=device)
            pool.fill_(float("nan") if poison else 0.0)
            self.kv.append(pool)
        self.states: dict[str, torch.Tensor] = {
            s.name: torch.zeros((max_requests, *s.shape), dtype=_STATE_DTYPES[s.dtype], device=device)
            for s in layout.states
        }

    def pages_of(self, cache_layer: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Key pages and value pages ``[pages, kv heads, page_size, head_dim]`` of one cache layer."""
        placed = self.layout.placement[cache_layer]
        if placed is None:
            raise KeyError(f"cache layer {cache_layer} holds no pages")
        group, local = placed
        return self.kv[group][local, 0], self.kv[group][local, 1]

    def zero_slots(self, slots: list[int]) -> None:
        if slots and self.states:
            index = torch.tensor(slots, dtype=torch.long, device=self.device)
            for t in self.states.values():
                t.index_fill_(0, index, 0)

    def poison_pages(self, freed: list[tuple[int, int]]) -> None:
        """Overwrite freed pages with NaN (tests: a read of a stale page then shows in the logits)."""
        if not (self.poison and freed):
            return
        for g in range(len(self.kv)):
            pages = [p for gi, p in freed if gi == g]
            if pages:
                index = torch.tensor(pages, dtype=torch.long, device=self.device)
                self.kv[g].index_fill_(2, index, float("nan"))

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv) + sum(
            t.numel() * t.element_size() for t in self.states.values())
