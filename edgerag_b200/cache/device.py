"""The tensors behind the cache manager: page pools per group and state records per slot.

One allocation per cache group, made once (the reference's arena: edgerag/serve/executor.py:76-83),
laid out ``[layer, k|v, page, kv head, offset, head_dim]`` so that one (layer, page, head) is a
contiguous ``page_size * head_dim`` run: the unit an attention kernel streams.  A group whose
values have another width than its keys (``KVGroupSpec.v_head_dim``) gets a key pool and a value
pool of their own, each ``[layer, page, kv head, offset, width]``.
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
        #: per group: (key pool, value pool, the dimension of each that counts pages)
        self._pools: list[tuple[torch.Tensor, torch.Tensor, int]] = []
        self.kv: list[torch.Tensor] = []         # the allocations themselves (one or two per group)
        fill = float("nan") if poison else 0.0
        for g, n in zip(layout.groups, num_pages):
            if g.value_dim == g.head_dim:
                pool = torch.empty((g.n_layers, 2, n, g.n_kv_heads, page_size, g.head_dim), dtype=dtype, device=device)
                pool.fill_(fill)
                self.kv.append(pool)
                self._pools.append((pool[:, 0], pool[:, 1], 1))
            else:
                keys = torch.empty((g.n_layers, n, g.n_kv_heads, page_size, g.head_dim), dtype=dtype, device=device)
                values = torch.empty((g.n_layers, n, g.n_kv_heads, page_size, g.value_dim), dtype=dtype, device=device)
                keys.fill_(fill), values.fill_(fill)
                self.kv += [keys, values]
                self._pools.append((keys, values, 1))
        self.states: dict[str, torch.Tensor] = {
            s.name: torch.zeros((max_requests, *s.shape), dtype=_STATE_DTYPES[s.dtype], device=device)
            for s in layout.states
        }

    def pages_of(self, cache_layer: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Key pages ``[pages, kv heads, page_size, head_dim]`` and value pages (the same shape, or
        ``v_head_dim`` wide where the group says so) of one cache layer."""
        placed = self.layout.placement[cache_layer]
        if placed is None:
            raise KeyError(f"cache layer {cache_layer} holds no pages")
        group, local = placed
        keys, values, _ = self._pools[group]
        return keys[local], values[local]

    def zero_slots(self, slots: list[int]) -> None:
        if slots and self.states:
            index = torch.tensor(slots, dtype=torch.long, device=self.device)
            for t in self.states.values():
                t.index_fill_(0, index, 0)

    def poison_pages(self, freed: list[tuple[int, int]]) -> None:
        """Overwrite freed pages with NaN (tests: a read of a stale page then shows in the logits)."""
        if not (self.poison and freed):
            return
        for g, (keys, values, page_dim) in enumerate(self._pools):
            pages = [p for gi, p in freed if gi == g]
            if pages:
                index = torch.tensor(pages, dtype=torch.long, device=self.device)
                keys.index_fill_(page_dim, index, float("nan"))
                values.index_fill_(page_dim, index, float("nan"))

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv) + sum(
            t.numel() * t.element_size() for t in self.states.values())
