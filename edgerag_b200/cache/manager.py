"""The cache manager: paged keys and values per cache group, block tables per request, state slots.

What the reference spreads over ``BlockTable`` (edgerag/cache/block_table.py:26-138),
``PagedKVCache`` (edgerag/cache/paged.py:40-261) and the arena of ``ModelExecutor``
(edgerag/serve/executor.py:76-83), re-cut for a batched step function:

* A **cache group** is a set of layers with the same needs (kv heads, head size, window).  Each
  group has pages of its own, an allocator of its own, and one block table per request.  The
  reference's only example of two groups is ``CompressedKVCache`` (edgerag/cache/compressed.py:49-68).
* A page holds ``page_size`` tokens of every layer of its group.  Token ``p`` of a request lives in
  page ``table[p // page_size]`` at offset ``p % page_size``; the token count is the only truth
  about length (edgerag/cache/block_table.py:60-79), and growth happens before the count advances,
  so a failed growth leaves the request untouched.
* Pages go back to the pool when the request is released, or, in a windowed group, as soon as no
  later query can see any key of the page.
* Beside the pages, every request holds one **state slot**: the index of a fixed-size record in
  each state tensor that a mixer registered (none for the Llama decoder).  Slots are zeroed when
  handed out.

The bookkeeping is tensor-free; ``DevicePools`` holds the tensors and is the only part that needs
a GPU.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .allocator import AllocatorError, OutOfPagesError, UnitAllocator

NO_PAGE = -1


@dataclass(frozen=True)
class KVGroupSpec:
    """Layers whose keys and values share page geometry."""

    n_layers: int
    n_kv_heads: int
    head_dim: int
    window: int = 0  # 0: every earlier key stays visible
    #: width of a cached value row when it differs from the key's (a mixer that caches keys and
    #: values of different sizes, or a single latent per token with ``v_head_dim = 0``); None: head_dim
    v_head_dim: int | None = None

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim

    def page_elements(self, page_size: int) -> int:
        """Elements one page holds over all layers of the group (keys and values)."""
        return self.n_layers * self.n_kv_heads * page_size * (self.head_dim + self.value_dim)


@dataclass(frozen=True)
class StateSpec:
    """A per-request record of fixed size kept by a mixer (``shape`` per request, float32 unless said)."""

    name: str
    shape: tuple[int, ...]
    dtype: str = "float32"


@dataclass
class CacheLayout:
    """What a model needs from the cache: its groups, where each cache layer lives, its states."""

    groups: list[KVGroupSpec] = field(default_factory=list)
    #: cache layer -> (group index, layer index inside the group); None for layers without pages
    placement: list[tuple[int, int] | None] = field(default_factory=list)
    states: list[StateSpec] = field(default_factory=list)

    def bytes_per_token(self, itemsize: int) -> int:
        """Bytes of cache one token takes over all groups (ignoring windows)."""
        return sum(g.page_elements(1) * itemsize for g in self.groups)


@dataclass
class BlockTable:
    """One request's pages in one group.  ``pages[i]`` is ``NO_PAGE`` once a window has passed page i."""

    pages: list[int] = field(default_factory=list)
    first_live: int = 0  # index of the first page not yet given back
    #: the same ids as an int32 array (capacity grows by doubling), for building batches without Python loops
    _array: np.ndarray = field(default_factory=lambda: np.zeros(16, np.int32), repr=False, compare=False)

    def extend(self, new_pages: list[int]) -> None:
        n = len(self.pages)
        if n + len(new_pages) > self._array.size:
            grown = np.zeros(max(2 * self._array.size, n + len(new_pages)), np.int32)
            grown[:n] = self._array[:n]
            self._array = grown
        self._array[n: n + len(new_pages)] = new_pages
        self.pages.extend(new_pages)

    def mark_released(self, index: int) -> None:
        self.pages[index] = NO_PAGE
        self._array[index] = NO_PAGE

    def array(self) -> np.ndarray:
        """Page ids as int32 (a view: do not write)."""
        return self._array[: len(self.pages)]


@dataclass
class RequestCache:
    """Everything the cache holds for one request."""

    request_id: object
    slot: int
    tables: list[BlockTable]
    num_tokens: int = 0


class CacheManager:
    """Pages, block tables and slots for all live requests.  No tensors: see ``DevicePools``."""

    def __init__(self, layout: CacheLayout, page_size: int, num_pages: int | list[int], max_requests: int) -> None:
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, got {page_size}")
        self.layout = layout
        self.page_size = page_size
        per_group = num_pages if isinstance(num_pages, list) else [num_pages] * len(layout.groups)
        if len(per_group) != len(layout.groups):
            raise ValueError("num_pages must give one count per cache group")
        self.pages = [UnitAllocator(n, "page") for n in per_group]
        self.slots = UnitAllocator(max_requests, "state slot")
        self.requests: dict[object, RequestCache] = {}
        #: pages freed since the last call of ``drain_freed`` (group, page): for poisoning in tests
        self._freed: list[tuple[int, int]] = []
        #: slots handed out since the last ``drain_new_slots``: their state records must be zeroed
        self._new_slots: list[int] = []

    # --- sizes ----------------------------------------------------------------------------------

    def pages_for(self, n_tokens: int) -> int:
        """ceil(n_tokens / page_size) (edgerag/cache/allocator.py:244-254)."""
        if n_tokens < 0:
            raise ValueError(f"negative token count {n_tokens}")
        return -(-n_tokens // self.page_size)

    def peak_pages(self, final_tokens: int, max_step_tokens: int) -> list[int]:
        """Upper bound, per group, of the pages a request holds at any time on its way to ``final_tokens``.

        A group without a window holds every page.  A windowed group holds the pages that the
        window and one step's new tokens can touch.
        """
        out = []
        for g in self.layout.groups:
            full = self.pages_for(final_tokens)
            if g.window > 0:
                span = g.window + max(1, max_step_tokens)
                out.append(min(full, self.pages_for(span) + 1))
            else:
                out.append(full)
        return out

    def free_pages(self) -> list[int]:
        return [a.num_free for a in self.pages]

    def held_pages(self, request_id: object) -> list[int]:
        rc = self.requests[request_id]
        return [len(t.pages) - t.first_live for t in rc.tables]   # released pages are exactly the first ones

    # --- life of a request ------------------------------------------------------------------------

    def admit(self, request_id: object) -> RequestCache:
        """Give the request a state slot and empty block tables."""
        if request_id in self.requests:
            raise AllocatorError(f"request {request_id!r} is already admitted")
        (slot,) = self.slots.allocate(1)
        rc = RequestCache(request_id, slot, [BlockTable() for _ in self.layout.groups])
        self.requests[request_id] = rc
        self._new_slots.append(slot)
        return rc

    def pages_to_grow(self, request_id: object, n_new: int) -> list[int]:
        """Pages each group must still allocate before ``n_new`` more tokens can be written."""
        rc = self.requests[request_id]
        need = self.pages_for(rc.num_tokens + n_new)
        return [max(0, need - len(t.pages)) for t in rc.tables]

    def can_grow(self, request_id: object, n_new: int) -> bool:
        return all(n <= a.num_free for n, a in zip(self.pages_to_grow(request_id, n_new), self.pages))

    def grow(self, request_id: object, n_new: int) -> None:
        """Make room for ``n_new`` more tokens in every group, or raise with nothing changed."""
        rc = self.requests[request_id]
        extra = self.pages_to_grow(request_id, n_new)
        for n, a in zip(extra, self.pages):
            if n > a.num_free:
                a.stats.failed_allocations += 1
                raise OutOfPagesError(
                    f"request {request_id!r} needs {n} more pages, {a.num_free} of {a.capacity} free")
        for n, a, t in zip(extra, self.pages, rc.tables):
            t.extend(a.allocate(n))

    def slots_for(self, request_id: object, n_new: int) -> list[np.ndarray]:
        """Per group, the flat cache slot ``page * page_size + offset`` of each of the next ``n_new`` tokens."""
        rc = self.requests[request_id]
        ps = self.page_size
        positions = np.arange(rc.num_tokens, rc.num_tokens + n_new, dtype=np.int64)
        out = []
        for t in rc.tables:
            pages = t.array()[positions // ps]
            if (pages == NO_PAGE).any():
                raise AllocatorError(f"request {request_id!r}: a position to write lies in a released page")
            out.append((pages.astype(np.int64) * ps + positions % ps).astype(np.int32))
        return out

    def advance(self, request_id: object, n_new: int) -> None:
        """Record ``n_new`` written tokens and give back pages that a window has passed."""
        rc = self.requests[request_id]
        need = self.pages_for(rc.num_tokens + n_new)
        if any(len(t.pages) < need for t in rc.tables):
            raise AllocatorError(f"request {request_id!r}: advance past its pages (grow first)")
        rc.num_tokens += n_new
        ps = self.page_size
        for gi, (g, t) in enumerate(zip(self.layout.groups, rc.tables)):
            if g.window <= 0:
                continue
            # A later query sits at position >= num_tokens and sees keys > position - window, so
            # keys <= num_tokens - window are dead; page i is dead when its last key is.
            dead_upto = rc.num_tokens - g.window
            while t.first_live < len(t.pages) and (t.first_live + 1) * ps - 1 <= dead_upto:
                page = t.pages[t.first_live]
                self.pages[gi].free([page])
                self._freed.append((gi, page))
                t.mark_released(t.first_live)
                t.first_live += 1

    def release(self, request_id: object) -> None:
        """Give back everything the request holds."""
        rc = self.requests.pop(request_id)
        for gi, t in enumerate(rc.tables):
            live = [p for p in t.pages if p != NO_PAGE]
            self.pages[gi].free(live)
            self._freed.extend((gi, p) for p in live)
            t.pages.clear()
        self.slots.free([rc.slot])

    # --- hooks for the device side ----------------------------------------------------------------

    def drain_freed(self) -> list[tuple[int, int]]:
        freed, self._freed = self._freed, []
        return freed

    def drain_new_slots(self) -> list[int]:
        slots, self._new_slots = self._new_slots, []
        return slots

    # --- checks -----------------------------------------------------------------------------------

    def check_invariants(self) -> None:
        """No page lost, held twice or free while held; every request's tables match its length."""
        for a in self.pages:
            a.check_invariants()
        self.slots.check_invariants()
        for gi, a in enumerate(self.pages):
            held = [p for rc in self.requests.values() for p in rc.tables[gi].pages if p != NO_PAGE]
            if len(set(held)) != len(held):
                raise AllocatorError(f"group {gi}: a page is held by two owners")
            if len(held) != a.num_used:
                raise AllocatorError(f"group {gi}: {a.num_used} pages used but {len(held)} in block tables")
            for p in held:
                if not a.is_held(p):
                    raise AllocatorError(f"group {gi}: page {p} is in a block table and free")
        slots = [rc.slot for rc in self.requests.values()]
        if len(set(slots)) != len(slots) or len(slots) != self.slots.num_used:
            raise AllocatorError("state slots and live requests disagree")
        for rc in self.requests.values():
            for t in rc.tables:
                if len(t.pages) < self.pages_for(rc.num_tokens):
                    raise AllocatorError(f"request {rc.request_id!r}: fewer pages than its tokens need")

    def to_dict(self) -> dict[str, object]:
        return {
            "page_size": self.page_size,
            "groups": [a.to_dict() for a in self.pages],
            "slots": self.slots.to_dict(),
            "live_requests": len(self.requests),
        }
