"""Iteration-level scheduler: admission, portions of prompts under a token budget, decoding,
finishing and freeing.  Tensor-free, like the reference's (edgerag/sched/scheduler.py:1-7).

Decisions, each with its counterpart in the reference:

* **Order within a step** (edgerag/sched/scheduler.py:144-174): requests that decode come first
  (one token each), then requests in the middle of a prompt (at most ``max_prefills_per_step``),
  then new admissions from the head of the FIFO queue; never out of order.
* **Portions**: a prefilling request contributes at most ``prefill_chunk_size`` tokens per step
  (edgerag/serve/executor.py:51-54,118-120), and all entries of a step together at most
  ``max_step_tokens``.  Progress is committed only after the step ran (``update``), so a step that
  failed fakes no progress (edgerag/sched/request.py:100-119).
* **Admission budgets the final size** (edgerag/sched/scheduler.py:124-136): prompt plus everything
  the request may generate.  Unlike the reference, which checks free pages but allocates lazily
  and can therefore over-commit across admissions (edgerag/sched/scheduler.py:165-166 against
  edgerag/serve/executor.py:124,151), the pages a running request has yet to take are counted as
  committed, so an admitted request can always finish.  ``reserve_pages`` plays the part of the
  reference's ``cow_reserve_blocks``.
* **When pages run out**: (1) at admission the request waits at the head of the queue
  (``admission_blocked``); (2) a request that can never fit (more pages than the pool has, or
  longer than ``max_model_len``) is rejected when it is added instead of waiting forever; (3) with
  ``overcommit`` (admission by current size) a step may lack pages: then the newest running
  requests are preempted, newest first, their pages freed, and they return to the *front* of the
  queue to be recomputed (prompt and generated tokens) when readmitted
  (edgerag/sched/scheduler.py:210-253).  Swapping to host memory is not built.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Any

from ..cache.manager import CacheManager
from .request import Request, RequestState


@dataclass
class SchedulerConfig:
    max_batch_size: int = 8
    prefill_chunk_size: int = 512
    max_prefills_per_step: int = 1
    #: tokens all entries of a step may hold together; None: chunk * prefills + batch size
    max_step_tokens: int | None = None
    reserve_pages: int = 0
    eos_token_id: int | None = None
    max_model_len: int | None = None
    overcommit: bool = False

    def __post_init__(self) -> None:
        if self.max_batch_size < 1 or self.prefill_chunk_size < 1 or self.max_prefills_per_step < 1:
            raise ValueError("max_batch_size, prefill_chunk_size and max_prefills_per_step must be >= 1")
        if self.max_step_tokens is None:
            self.max_step_tokens = self.prefill_chunk_size * self.max_prefills_per_step + self.max_batch_size
        if self.max_step_tokens < 1:
            raise ValueError("max_step_tokens must be >= 1")


@dataclass
class SchedulerStats:
    steps: int = 0
    admitted: int = 0
    finished: int = 0
    rejected: int = 0
    preempted: int = 0
    prefill_portions: int = 0
    decode_tokens: int = 0
    admission_blocked: int = 0

    def to_dict(self) -> dict[str, int]:
        return dict(self.__dict__)


@dataclass
class ScheduledEntry:
    request: Request
    start: int          # index into prompt + generated of the first token fed
    n_tokens: int
    from_embeds: bool
    samples: bool       # the portion reaches the end of the known tokens: its last logits are sampled

    @property
    def is_decode(self) -> bool:
        return self.n_tokens == 1 and self.samples


@dataclass
class Batch:
    step: int
    entries: list[ScheduledEntry] = field(default_factory=list)

    @property
    def is_empty(self) -> bool:
        return not self.entries

    @property
    def n_tokens(self) -> int:
        return sum(e.n_tokens for e in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, config: SchedulerConfig | None = None) -> None:
        self.cache = cache
        self.config = config or SchedulerConfig()
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.finished: list[Request] = []
        self.step_index = 0
        self.stats = SchedulerStats()

    # --- queue ------------------------------------------------------------------------------------

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _peak(self, request: Request) -> list[int]:
        tokens = request.total_tokens + 1 if self.config.overcommit else request.final_tokens
        return self.cache.peak_pages(tokens, self.config.prefill_chunk_size)

    def add_request(self, request: Request) -> bool:
        """Queue a request, or reject it now if it can never run.  Returns whether it was queued."""
        request.arrival_step = self.step_index
        cfg = self.config
        reason = None
        if request.prompt_len < 1:
            reason = "empty_prompt"
        elif cfg.max_model_len is not None and request.final_tokens > cfg.max_model_len:
            reason = "too_long"
        else:
            peak = self.cache.peak_pages(request.final_tokens, cfg.prefill_chunk_size)
            if any(p > a.capacity - cfg.reserve_pages for p, a in zip(peak, self.cache.pages)):
                reason = "exceeds_pool"
        if reason:
            self._reject(request, reason)
            return False
        request.state = RequestState.WAITING
        self.waiting.append(request)
        return True

    def _reject(self, request: Request, reason: str) -> None:
        request.state = RequestState.REJECTED
        request.finish_reason = reason
        request.finished_step = self.step_index
        self.finished.append(request)
        self.stats.rejected += 1

    # --- accounting ---------------------------------------------------------------------------------

    def _committed(self) -> list[int]:
        """Pages, per group, that running requests are still entitled to take."""
        total = [0] * len(self.cache.pages)
        for r in self.running:
            held = self.cache.held_pages(r.request_id)
            for g, (p, h) in enumerate(zip(self._peak(r), held)):
                total[g] += max(0, p - h)
        return total

    def available_pages(self) -> list[int]:
        """Pages a new admission may count on (edgerag/sched/scheduler.py:120-123)."""
        return [max(0, f - c - self.config.reserve_pages)
                for f, c in zip(self.cache.free_pages(), self._committed())]

    # --- the decision ---------------------------------------------------------------------------------

    def _entry_for(self, request: Request, limit: int) -> ScheduledEntry:
        start, n, from_embeds = request.next_portion(limit)
        return ScheduledEntry(request, start, n, from_embeds, samples=(start + n == request.total_tokens))

    def schedule(self) -> Batch:
        cfg = self.config
        batch = Batch(self.step_index)
        budget = cfg.max_step_tokens
        n_prefills = 0

        decoding = [r for r in self.running if r.pending == 1]
        prefilling = [r for r in self.running if r.pending > 1]
        for r in decoding:
            if budget < 1:
                break
            batch.entries.append(self._entry_for(r, 1))
            budget -= 1
        for r in prefilling:
            if n_prefills >= cfg.max_prefills_per_step or budget < 1:
                break
            e = self._entry_for(r, min(cfg.prefill_chunk_size, budget))
            batch.entries.append(e)
            budget -= e.n_tokens
            n_prefills += 1

        self._make_room(batch)

        while (self.waiting and len(self.running) < cfg.max_batch_size
               and n_prefills < cfg.max_prefills_per_step and budget >= 1 and self.cache.slots.num_free > 0):
            r = self.waiting[0]
            if any(p > a for p, a in zip(self._peak(r), self.available_pages())):
                self.stats.admission_blocked += 1
                break
            self.waiting.popleft()
            self.cache.admit(r.request_id)
            r.admitted_step = self.step_index
            r.state = RequestState.PREFILLING if r.pending > 1 else RequestState.DECODING
            self.running.append(r)
            self.stats.admitted += 1
            e = self._entry_for(r, min(cfg.prefill_chunk_size, budget))
            batch.entries.append(e)
            budget -= e.n_tokens
            n_prefills += 1
        return batch

    def _make_room(self, batch: Batch) -> None:
        """Preempt the newest running requests until the entries' pages fit (overcommit only)."""
        while batch.entries:
            need = [0] * len(self.cache.pages)
            for e in batch.entries:
                for g, n in enumerate(self.cache.pages_to_grow(e.request.request_id, e.n_tokens)):
                    need[g] += n
            if all(n <= f for n, f in zip(need, self.cache.free_pages())):
                return
            victim = self.running[-1]
            if len(self.running) == 1:
                # Alone and still too large for the pool: it can never finish.
                self._release(victim)
                self.running.remove(victim)
                self._reject(victim, "out_of_pages")
                batch.entries = [e for e in batch.entries if e.request is not victim]
                return
            self.preempt(victim)
            batch.entries = [e for e in batch.entries if e.request is not victim]

    def preempt(self, request: Request) -> None:
        """Free a running request's pages and send it to the front of the queue for recomputation."""
        self._release(request)
        self.running.remove(request)
        request.num_computed = 0
        request.state = RequestState.WAITING
        request.preemptions += 1
        self.waiting.appendleft(request)
        self.stats.preempted += 1

    def _release(self, request: Request) -> None:
        if request.request_id in self.cache.requests:
            self.cache.release(request.request_id)

    # --- after the step ---------------------------------------------------------------------------------

    def update(self, batch: Batch, new_tokens: dict[str, int]) -> list[Request]:
        """Commit a step that ran: advance every entry, append sampled tokens, finish and free.
        Entries of requests that have finished since the step was launched are skipped.

        Returns the requests that finished in this step.
        """
        done = []
        for e in batch.entries:
            r = e.request
            if r.is_finished:
                continue        # launched ahead for a request that stopped in the step before: dropped
            r.num_computed += e.n_tokens
            if e.is_decode:
                self.stats.decode_tokens += 1
            else:
                self.stats.prefill_portions += 1
            if e.samples:
                token = new_tokens[r.request_id]
                if r.first_token_step is None:
                    r.first_token_step = self.step_index
                r.generated_token_ids.append(int(token))
                if r.should_stop(self.config.eos_token_id):
                    eos = self.config.eos_token_id
                    r.finish_reason = "stop" if (eos is not None and token == eos) else "length"
                    self.finish(r)
                    done.append(r)
                    continue
            r.state = RequestState.PREFILLING if r.pending > 1 else RequestState.DECODING
        self.step_index += 1
        self.stats.steps += 1
        return done

    def finish(self, request: Request) -> None:
        """edgerag/sched/scheduler.py:193-202: mark finished, free its pages and slot at once."""
        request.state = RequestState.FINISHED
        request.finished_step = self.step_index
        self._release(request)
        if request in self.running:
            self.running.remove(request)
        self.finished.append(request)
        self.stats.finished += 1

    def abort(self, request: Request, reason: str = "aborted") -> None:
        """Fail a request wherever it is (the engine's error path, edgerag/serve/engine.py:235-241)."""
        if request in self.waiting:
            self.waiting.remove(request)
        request.finish_reason = reason
        self.finish(request)

    def to_dict(self) -> dict[str, Any]:
        return {"step": self.step_index, "waiting": len(self.waiting), "running": len(self.running),
                "finished": len(self.finished), "free_pages": self.cache.free_pages(),
                "available_for_admission": self.available_pages(), "stats": self.stats.to_dict()}
