"""The step function: one ragged batch of (request, its next tokens) through the model, from the cache.

The reference's ``ModelExecutor.execute`` (edgerag/serve/executor.py:112-156) runs every request of
a batch as a forward pass of its own with batch size 1.  Here all entries of a step form **one**
batch: portions of prompts of any length beside single decoded tokens, flattened to ``T`` tokens
with, per token, its id (or embedding row), logical position, sequence and cache slot, and per
sequence a block table.  Only the tokens given are run; everything earlier comes from the cache.
The result is the float32 logits at the places asked for, in the order of the entries and of
``want`` inside each entry; sampling sits above (the reference takes the argmax inside the
executor, edgerag/serve/executor.py:136,154).

Positions are logical and continue from the request's cached length (edgerag/core/model.py:112-120).
Entries with a single token are placed first inside the batch so that the split-KV decode kernel
and the row kernel each see a contiguous range; the caller's order is restored in the result.
"""

from __future__ import annotations

import gc
from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.device import DevicePools
from ..cache.manager import CacheManager, OutOfPagesError
from ..ops import kernels


_ITEMSIZE = {torch.float32: 4, torch.bfloat16: 2, torch.int32: 4, torch.int64: 8, torch.uint8: 1, torch.float16: 2}


class StepError(ValueError):
    """A step was asked for that cannot run (unknown request, bad ids, no room in the batch)."""


@dataclass
class StepEntry:
    """The next tokens of one request: ids, or rows of embeddings ``[n, hidden]``, or ``fed_back``:
    one token that is still on the device, row ``fed_back`` of the runner's ``feedback`` tensor
    (what the sampler wrote for the step before).  Exactly one of the three."""

    request_id: object
    tokens: list[int] | None = None
    embeds: torch.Tensor | None = None
    want: list[int] = field(default_factory=list)
    fed_back: int | None = None

    @property
    def n_tokens(self) -> int:
        if self.fed_back is not None:
            return 1
        return len(self.tokens) if self.embeds is None else int(self.embeds.shape[0])


class Workspace:
    """Named scratch buffers that keep their address from step to step (they only ever grow)."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self._bufs: dict[str, torch.Tensor] = {}
        self._views: dict[tuple, torch.Tensor] = {}
        #: called before a buffer that CUDA graphs may point at is replaced by a larger one
        self.on_move = None

    def get(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        key = (name, shape, dtype)
        view = self._views.get(key)
        if view is not None:
            return view
        need = int(np.prod(shape, dtype=np.int64)) * _ITEMSIZE[dtype]
        buf = self._bufs.get(name)
        if buf is None or buf.numel() < need:
            if buf is not None and self.on_move is not None:
                self.on_move()
            buf = torch.empty(max(need, 256), dtype=torch.uint8, device=self.device)
            self._bufs[name] = buf
            self._views = {k: v for k, v in self._views.items() if k[0] != name}
        view = buf[:need].view(dtype).view(shape)
        self._views[key] = view
        return view

    def nbytes(self) -> int:
        return sum(b.numel() for b in self._bufs.values())


class StepContext:
    """What every part sees of one step.  Device tensors are views of one uploaded int32 buffer."""

    def __init__(self, runner: "ModelRunner") -> None:
        self._runner = runner
        self.page_size = runner.cache.page_size
        self.dtype = runner.dtype
        #: parts choose launch shapes that do not depend on the batch (a request's results are then the
        #: same bits whatever shares its step, at some cost in speed)
        self.batch_invariant = runner.batch_invariant
        self.status = runner.status
        self.n_tokens = self.n_seqs = self.n_decode = self.n_wanted = self.n_fed_back = 0
        self.n_wanted_real = 0                       # wanted rows that belong to entries (the others to filler rows)
        self.token_ids = self.embed_row = self.positions = self.seq_of_token = None
        self.token_of_seq = self.want_rows = self.state_slots = self.seq_starts = None
        self.embeds: torch.Tensor | None = None
        self.max_pages = 1
        self.bound_pages, self.granule_pages = 4, 1
        self.graph_key: tuple | None = None          # set when the step has the fixed layout of a CUDA graph
        self.slots: list[torch.Tensor] = []
        self.block_tables: list[torch.Tensor] = []
        #: host copies for parts that size launches or loop over sequences
        self.host_q_len: list[int] = []
        self.host_positions_last: list[int] = []   # position of each sequence's last token of the step
        self.host_state_slots: list[int] = []

    def buf(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        return self._runner.workspace.get(name, shape, dtype)

    def pages_of(self, cache_layer: int) -> tuple[torch.Tensor, torch.Tensor]:
        return self._runner.pools.pages_of(cache_layer)

    def group_of(self, cache_layer: int) -> int:
        return self._runner.cache.layout.placement[cache_layer][0]

    def state(self, name: str, cache_layer: int) -> torch.Tensor:
        """The state tensor ``[slots, ...]`` a mixer registered under ``name`` for a cache layer."""
        return self._runner.pools.states[f"{name}@{cache_layer}"]

    def max_keys_bound(self) -> int:
        """A bound on the longest context of the batch that steps of one captured layout share: its pages
        rounded up to a quarter of their power-of-two bucket (``kernels.context_bound``), in tokens."""
        return self.bound_pages * self.page_size

    def keys_granule(self) -> int:
        """The step of ``max_keys_bound`` in tokens: the batch's longest context lies within one granule below the bound."""
        return self.granule_pages * self.page_size

    def decode_splits(self, window: int, split_keys: int = kernels.DECODE_SPLIT_KEYS) -> int:
        """Largest number of key splits any single-token sequence of the batch has."""
        if self.graph_key is not None:   # a captured layout: the bound must hold for every replay
            bound = -(-(self.bound_pages * self.page_size) // split_keys)
            return bound if window <= 0 else min(bound, window // split_keys + 2)
        most = 1
        for pos in self.host_positions_last[: self.n_decode]:
            lo = max(0, pos - window + 1) if window > 0 else 0
            most = max(most, pos // split_keys - lo // split_keys + 1)
        return most


def _fill_to(n: int) -> int:
    """The size that ``n`` single-token rows of a captured step are filled up to: the next power of two up to 8, then the next multiple of 8."""
    return 1 << (n - 1).bit_length() if n <= 8 else -(-n // 8) * 8


class ModelRunner:
    """Owns the model, the cache and the scratch of one device, and runs steps on them."""

    def __init__(self, model, cache: CacheManager, pools: DevicePools, max_step_tokens: int,
                 check_status: bool = False, cuda_graphs: bool = False, batch_invariant: bool = False,
                 pad_decodes: bool = True, tune_products: bool = False) -> None:
        self.model = model
        self.tune_products = bool(tune_products)     # see EngineOptions.tune_products
        self.batch_invariant = bool(batch_invariant)
        #: steps whose tokens are all ids get their single-token sequences (and their wanted rows) filled up
        #: to the next of a few sizes with rows that read one cached key, write nothing and are dropped
        #: again, so that the number of running requests, which changes all the time in serving, changes
        #: the layout (and with it the captured graph) only now and then; done whether or not graphs are
        #: on, so that turning them on changes no bit
        self.pad_decodes = bool(pad_decodes)
        self.cache = cache
        self.pools = pools
        self.device = pools.device
        self.dtype = model.dtype
        self.max_step_tokens = max_step_tokens
        self.check_status = check_status
        self.workspace = Workspace(self.device)
        self.workspace.on_move = self.drop_graphs
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        #: int32 device tensor that entries with ``fed_back`` take their token from (set by the caller)
        self.feedback: torch.Tensor | None = None
        #: host copy of the status word, refreshed asynchronously at the end of every step
        self._status_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        self._meta_dev: torch.Tensor | None = None
        #: pinned staging buffers, used in turn; each waits for its last upload before it is rewritten
        self._meta_host: list[torch.Tensor | None] = [None] * 4
        self._meta_event: list[torch.cuda.Event | None] = [None] * 4
        self._meta_turn = 0
        self.steps_run = 0
        self.h2d_bytes_last = 0
        #: steps are captured in CUDA graphs, one per (single tokens, portion lengths, page bucket, wanted
        #: rows), the second time a layout is seen; only models whose parts all declare ``graph_safe``
        self.graphs_enabled = bool(cuda_graphs) and bool(getattr(model, "graph_safe", False))
        self.max_graphs = 512
        self._graphs: dict[tuple, tuple] = {}
        self._graph_seen: dict[tuple, int] = {}
        self.graph_replays = 0
        if self.graphs_enabled:
            self._meta_dev = torch.empty(1 << 20, dtype=torch.int32, device=self.device)

    # --- metadata buffer --------------------------------------------------------------------------

    def _upload(self, flat: np.ndarray) -> torch.Tensor:
        """Copy the step's int32 metadata to the device through pinned memory (one transfer)."""
        n = flat.size
        if self._meta_dev is None or self._meta_dev.numel() < n:
            self.drop_graphs()
            self._meta_dev = torch.empty(max(4096, 2 * n), dtype=torch.int32, device=self.device)
        i = self._meta_turn = (self._meta_turn + 1) % len(self._meta_host)
        if self._meta_event[i] is not None:
            self._meta_event[i].synchronize()
        if self._meta_host[i] is None or self._meta_host[i].numel() < n:
            self._meta_host[i] = torch.empty(max(4096, 2 * n), dtype=torch.int32, pin_memory=True)
        host = self._meta_host[i]
        host[:n].copy_(torch.from_numpy(flat))
        self._meta_dev[:n].copy_(host[:n], non_blocking=True)
        if self._meta_event[i] is None:
            self._meta_event[i] = torch.cuda.Event()
        self._meta_event[i].record()
        self.h2d_bytes_last = 4 * n
        return self._meta_dev

    # --- the step ---------------------------------------------------------------------------------

    def prepare(self, entries: list[StepEntry]) -> tuple[StepContext, list[StepEntry]]:
        """Validate, make room in the cache, and upload the batch's metadata.  Nothing is run yet."""
        if not entries:
            raise StepError("a step needs at least one entry")
        vocab, hidden = self.model.vocab_size, self.model.hidden_size
        seen = set()
        for e in entries:
            if e.request_id not in self.cache.requests:
                raise StepError(f"request {e.request_id!r} is not admitted")
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if (e.tokens is not None) + (e.embeds is not None) + (e.fed_back is not None) != 1:
                raise StepError(f"request {e.request_id!r}: pass exactly one of tokens, embeds or fed_back")
            if e.fed_back is not None and (self.feedback is None or not 0 <= e.fed_back < self.feedback.numel()):
                raise StepError(f"request {e.request_id!r}: no fed-back token in row {e.fed_back}")
            n = e.n_tokens
            if n <= 0:
                raise StepError(f"request {e.request_id!r}: an entry needs at least one token")
            if e.embeds is not None and (e.embeds.dim() != 2 or e.embeds.shape[1] != hidden):
                raise StepError(f"request {e.request_id!r}: embeds must be [n, {hidden}]")
            if e.tokens is not None and not all(0 <= int(t) < vocab for t in e.tokens):
                raise StepError(f"request {e.request_id!r}: a token id is outside [0, {vocab})")
            if any(not 0 <= int(w) < n for w in e.want):
                raise StepError(f"request {e.request_id!r}: a wanted place is outside its {n} tokens")
        total = sum(e.n_tokens for e in entries)
        if total > self.max_step_tokens:
            raise StepError(f"{total} tokens exceed the step limit of {self.max_step_tokens}")

        # Room in every group for all entries, or nothing changes.
        n_groups = len(self.cache.layout.groups)
        need = [0] * n_groups
        for e in entries:
            for g, n in enumerate(self.cache.pages_to_grow(e.request_id, e.n_tokens)):
                need[g] += n
        free = self.cache.free_pages()
        if any(n > f for n, f in zip(need, free)):
            raise OutOfPagesError(f"step needs {need} more pages per group, {free} free")
        for e in entries:
            self.cache.grow(e.request_id, e.n_tokens)

        # Single-token entries first; a stable order otherwise.
        order = sorted(range(len(entries)), key=lambda i: (entries[i].n_tokens != 1, i))
        ordered = [entries[i] for i in order]
        n_decode = sum(1 for e in ordered if e.n_tokens == 1)
        # A step whose layout is fully described by a small key can be replayed from a CUDA graph:
        # single tokens, and portions of prompts given as ids (their lengths are part of the key).
        graphable = self.graphs_enabled and all(e.embeds is None for e in ordered)
        # Filler rows between the single tokens and the portions (None in `rows`): see `pad_decodes`.
        n_fill = 0
        if self.pad_decodes and n_decode and all(e.embeds is None for e in ordered) and not self.cache.layout.states:
            n_fill = _fill_to(n_decode) - n_decode
            if total + n_fill > self.max_step_tokens:
                n_fill = 0
        rows: list[StepEntry | None] = ordered[:n_decode] + [None] * n_fill + ordered[n_decode:]
        origins = order[:n_decode] + [-1] * n_fill + order[n_decode:]
        total += n_fill
        n_decode += n_fill
        n_seqs = len(rows)
        ps = self.cache.page_size

        token_ids = np.zeros(total, np.int32)
        embed_row = np.full(total, -1, np.int32)
        positions = np.zeros(total, np.int32)
        seq_of_token = np.zeros(total, np.int32)
        slots = np.full((n_groups, total), -1, np.int32)
        token_of_seq = np.zeros(n_seqs, np.int32)
        seq_starts = np.zeros(n_seqs + 1, np.int32)
        state_slots = np.zeros(n_seqs, np.int32)
        max_pages = 1
        for e in ordered:
            rc = self.cache.requests[e.request_id]
            max_pages = max(max_pages, max((len(t.pages) for t in rc.tables), default=1))
        bound_pages, granule_pages = kernels.context_bound(max_pages)
        if graphable:
            # a captured step has a fixed layout: block tables padded to a power of two of pages
            max_pages = max(4, 1 << (max_pages - 1).bit_length())
        tables = np.zeros((n_groups, n_seqs, max_pages), np.int32)
        want_of_entry: dict[int, list[int]] = {}
        embed_chunks: list[torch.Tensor] = []
        n_embed_rows = 0
        ctx = StepContext(self)
        t0 = 0
        for s, (orig, e) in enumerate(zip(origins, rows)):
            if e is None:
                # a filler: token 0 at position 0 of a sequence whose table names page 0 only; it reads that
                # page's first key (whatever it holds: the row's results go nowhere) and has no cache slot
                seq_of_token[t0] = s
                token_of_seq[s] = t0
                seq_starts[s + 1] = t0 + 1
                ctx.host_q_len.append(1)
                ctx.host_positions_last.append(0)
                ctx.host_state_slots.append(0)
                t0 += 1
                continue
            rc = self.cache.requests[e.request_id]
            n = e.n_tokens
            past = rc.num_tokens
            sl = slice(t0, t0 + n)
            positions[sl] = np.arange(past, past + n, dtype=np.int32)
            seq_of_token[sl] = s
            if e.fed_back is not None:
                token_ids[sl] = -1 - e.fed_back
            elif e.embeds is None:
                token_ids[sl] = np.asarray(e.tokens, dtype=np.int32)
            else:
                embed_row[sl] = np.arange(n_embed_rows, n_embed_rows + n, dtype=np.int32)
                embed_chunks.append(e.embeds)
                n_embed_rows += n
            for g, row in enumerate(self.cache.slots_for(e.request_id, n)):
                slots[g, sl] = row
                pages = rc.tables[g].array()
                tables[g, s, : pages.size] = np.maximum(pages, 0)     # released pages are never read: any id does
            token_of_seq[s] = t0
            seq_starts[s + 1] = t0 + n
            state_slots[s] = rc.slot
            want_of_entry[orig] = [t0 + int(w) for w in e.want]
            ctx.host_q_len.append(n)
            ctx.host_positions_last.append(past + n - 1)
            ctx.host_state_slots.append(rc.slot)
            t0 += n
        wanted = [r for i in range(len(entries)) for r in want_of_entry[i]]
        n_wanted_real = len(wanted)
        if n_fill and wanted:                  # the wanted rows are filled up the same way (with the first of them again)
            wanted += [wanted[0]] * (_fill_to(len(wanted)) - len(wanted))
        want_rows = np.asarray(wanted, dtype=np.int32)

        pieces = [token_ids, embed_row, positions, seq_of_token, slots.reshape(-1), token_of_seq, seq_starts,
                  state_slots, want_rows, tables.reshape(-1)]
        flat = np.concatenate(pieces)
        dev = self._upload(flat)
        views, off = [], 0
        for p in pieces:
            views.append(dev[off: off + p.size])
            off += p.size
        (ctx.token_ids, ctx.embed_row, ctx.positions, ctx.seq_of_token, slots_d, ctx.token_of_seq, ctx.seq_starts,
         ctx.state_slots, ctx.want_rows, tables_d) = views
        ctx.slots = [slots_d[g * total: (g + 1) * total] for g in range(n_groups)]
        per = n_seqs * max_pages
        ctx.block_tables = [tables_d[g * per: (g + 1) * per].view(n_seqs, max_pages) for g in range(n_groups)]
        ctx.n_tokens, ctx.n_seqs, ctx.n_decode, ctx.n_wanted = total, n_seqs, n_decode, int(want_rows.size)
        ctx.n_wanted_real = n_wanted_real
        ctx.max_pages = max_pages
        ctx.bound_pages, ctx.granule_pages = bound_pages, granule_pages
        ctx.n_fed_back = sum(1 for e in ordered if e.fed_back is not None)
        if graphable:
            ctx.graph_key = (n_decode, tuple(e.n_tokens for e in ordered[n_decode - n_fill:]), max_pages, bound_pages,
                             int(want_rows.size))
        if embed_chunks:
            ctx.embeds = torch.cat([c.to(device=self.device, dtype=self.dtype, non_blocking=True)
                                    for c in embed_chunks], dim=0).contiguous()
        return ctx, ordered

    def finish(self, ordered: list[StepEntry]) -> None:
        """Count the step's tokens as written and hand back what windows have passed."""
        for e in ordered:
            self.cache.advance(e.request_id, e.n_tokens)

    @torch.inference_mode()
    def step(self, entries: list[StepEntry]) -> torch.Tensor | None:
        """Run one batch.  Returns float32 logits ``[wanted, vocab]`` (a view of a buffer that the
        next step overwrites), or ``None`` when nothing was wanted."""
        self.raise_if_flagged()
        self.pools.zero_slots(self.cache.drain_new_slots())
        # pages given back since the last step are overwritten before any of them is handed out again
        self.pools.poison_pages(self.cache.drain_freed())
        ctx, ordered = self.prepare(entries)
        if self.dtype == torch.bfloat16:
            kernels.linear_status_word(self.status)      # (the products report to this runner's word)
        if ctx.n_fed_back:
            kernels.resolve_ids(ctx.token_ids, self.feedback, self.dtype)
        logits = self._forward(ctx)
        if logits is not None and ctx.n_wanted_real < ctx.n_wanted:
            logits = logits[: ctx.n_wanted_real]          # (the rest belongs to filler rows)
        self.finish(ordered)
        self.steps_run += 1
        self._status_host.copy_(self.status, non_blocking=True)
        if self.check_status:
            torch.cuda.current_stream().synchronize()
            self.raise_if_flagged()
        return logits

    def raise_if_flagged(self) -> None:
        """Raise if a kernel of an earlier step reported a fault (checked from the pinned host copy of
        the status word, so callers that synchronise anyway pay nothing extra)."""
        code = int(self._status_host[0])
        if code:
            # Steps that are still on the device (one launched ahead) would copy the same code to the
            # host once more after it has been cleared here: let them finish first.
            torch.cuda.current_stream().synchronize()
            self.status.zero_()
            self._status_host.zero_()
            kernels.reset_split_counters()      # a block that gave up did not count itself among its sequence's splits
            if code >= 1000000:
                raise StepError(f"an attention kernel gave up (code {code}: 1xxxxxx prefill wait, 2xxxxxx decode "
                                "wait, 3000000 shared-memory alignment, 4xxxxxx a wait of a product for few rows); "
                                "the step's results are not valid")
            raise StepError(f"a kernel flagged token {code - 1} of the batch (id or row out of range)")

    def drop_graphs(self) -> None:
        """Forget every captured graph (a buffer they point at is about to move); they are captured again on demand."""
        self._graphs.clear()
        self._graph_seen.clear()

    def _forward(self, ctx: StepContext) -> torch.Tensor | None:
        """Run the model eagerly, or replay the CUDA graph captured for this step's layout.

        A layout is captured the second time it is seen (the first run sizes every scratch buffer).
        The graph holds the kernels' arguments; what changes from step to step (ids, positions,
        slots, block tables, wanted rows) lives in the metadata buffer at fixed offsets.
        """
        key = ctx.graph_key
        if key is None:
            return self.model.forward(ctx)
        hit = self._graphs.get(key)
        if hit is not None:
            hit[0].replay()
            self.graph_replays += 1
            kernels.launch_counts["own"] += hit[2]
            return hit[1]
        seen = self._graph_seen.get(key, 0)
        if len(self._graph_seen) > 8192:
            self._graph_seen.clear()
        self._graph_seen[key] = seen + 1
        capture = seen >= 1 and len(self._graphs) < self.max_graphs
        # The layout has come back and its graph will fix the library's algorithms for every replay: where
        # asked for, the run before the capture lets the library's proposals for its large products be timed once.
        tune = self.tune_products and capture and ctx.n_tokens >= kernels.LINEAR_TUNE_FROM_ROWS
        if tune:
            kernels.linear_tune(self.dtype, True)
        try:
            logits = self.model.forward(ctx)
        finally:
            if tune:
                kernels.linear_tune(self.dtype, False)
        if capture:
            graph = torch.cuda.CUDAGraph()
            before = kernels.launch_counts["own"]
            # No cyclic garbage collection while the stream captures: a collector run could destroy
            # tensors or graphs of an engine that is no longer referenced, which is not permitted
            # during a capture and would invalidate it.
            collecting = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph):
                    captured = self.model.forward(ctx)
            finally:
                if collecting:
                    gc.enable()
            own = kernels.launch_counts["own"] - before
            kernels.launch_counts["own"] = before       # capturing launched nothing
            self._graphs[key] = (graph, captured, own)
        return logits

    # --- requests ---------------------------------------------------------------------------------

    def admit(self, request_id: object) -> None:
        self.cache.admit(request_id)

    def release(self, request_id: object) -> None:
        self.cache.release(request_id)
