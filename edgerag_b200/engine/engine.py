"""The Python entry point: a model folder in, generated tokens out.

Assembly follows the reference's ``build_stack`` (bench/serving.py:159-279): configuration and
weights, one page pool sized from a block count or a memory budget, a scheduler over it, the step
function under it.  Driving follows the threadless loop of the reference's tests
(tests/test_executor.py:54-70): ``schedule -> execute -> bookkeeping`` per step, without the worker
thread and queues of ``InferenceEngine`` (edgerag/serve/engine.py:107-281), which belong to its
HTTP server.

    engine = Engine.from_pretrained("model_dir", dtype="bfloat16")
    outputs = engine.generate([[1, 2, 3]], SamplingParams(max_new_tokens=16))
"""

from __future__ import annotations

import json
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Iterator

import torch

from ..cache.device import DevicePools
from ..cache.manager import CacheManager, OutOfPagesError
from ..config.registry import architecture_of, read_model_folder
from ..models.decoder import DecoderModel
from ..sampling.params import SamplingParams
from ..sampling.sampler import PendingTokens, Sampler
from ..weights.loader import load_safetensors, random_tensors
from .request import Request, RequestState
from .scheduler import Batch, ScheduledEntry, Scheduler, SchedulerConfig
from .step import ModelRunner, StepEntry

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}
GIB = 1024 ** 3


def resolve_dtype(dtype: str | torch.dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {dtype} is not bfloat16 or float32")
        return dtype
    try:
        return DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype {dtype!r} is not one of {sorted(DTYPES)}") from None


def require_cuda(device: str | torch.device) -> torch.device:
    """The engine has no CPU path: fail with a clear message instead of falling back."""
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError(f"edgerag_b200 runs on a CUDA device only; asked for {device}, "
                           f"cuda available: {torch.cuda.is_available()}")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


@dataclass
class EngineOptions:
    """Engine knobs.  Names follow the reference's CLI and ``SchedulerConfig`` where it has them
    (scripts/serve_rag.py:104-131, edgerag/sched/scheduler.py:40-49)."""

    dtype: str | torch.dtype = "bfloat16"
    device: str = "cuda:0"
    block_size: int = 16                # tokens per cache page
    num_blocks: int | None = None       # pages in the pool; None: size it from the budget or fraction
    budget_gib: float | None = None     # total device memory the engine may use (weights included)
    kv_fraction: float = 0.8            # else: this share of the memory that is free after loading
    max_batch_size: int = 8
    chunk_size: int = 512               # prompt tokens per request per step
    max_prefills_per_step: int = 1
    max_step_tokens: int | None = None
    max_model_len: int | None = None
    reserve_blocks: int = 0
    eos_token_id: int | None = None
    overcommit: bool = False
    seed: int = 0
    cuda_graphs: bool = True
    #: launch the next decoding step before this step's tokens have reached the host (they are fed
    #: back on the device); what ``step`` returns is then one step behind what the GPU is running
    lookahead: bool = True
    poison_freed_pages: bool = False    # tests: NaN in free pages, so a stale read shows
    #: launch shapes that do not depend on the batch (decode attention always in splits of 512 keys with
    #: the default grouping of heads): up to 16 single-token rows a request's logits are then the same
    #: bits whatever shares its step; off, the attention kernel's shape follows the batch, which is
    #: faster for small batches and short contexts
    batch_invariant: bool = False
    #: captured steps fill their single-token rows up to the next of a few sizes (1, 2, 4, 8, 16, 24, ...), so
    #: that a change in the number of running requests seldom needs another graph
    pad_decodes: bool = True
    #: before a step's layout is captured into a CUDA graph, let the library's proposals for its products of
    #: 1,024 rows or more be timed against each other once (the fastest stays for the process).  A trial
    #: costs tens of milliseconds (every proposal is a kernel the library has to load): it pays where the same
    #: large steps run many hundreds of times (prompts served in portions of a fixed size: 5 % of a 2,048-token
    #: step), and costs where layouts change all the time, so it is off unless asked for
    tune_products: bool = False


@dataclass
class TokenEvent:
    """One generated token (edgerag/serve/engine.py:43-56)."""

    request_id: str
    token_id: int
    index: int
    finished: bool
    finish_reason: str | None = None


@dataclass
class _Launched:
    """A step on the device: its batch, the entries whose last logits are sampled, and the ids on their way."""

    batch: Batch
    sampled: list[ScheduledEntry]
    pending: PendingTokens | None


class Engine:
    def __init__(self, model: DecoderModel, config: Any, options: EngineOptions) -> None:
        self.model = model
        self.config = config
        self.options = options
        self.device = model.device
        self.dtype = model.dtype
        layout = model.cache_layout
        itemsize = 2 if self.dtype == torch.bfloat16 else 4
        max_len = options.max_model_len or getattr(config, "max_position_embeddings", None) or 8192
        self.max_model_len = max_len
        if options.num_blocks is not None:
            num_pages = options.num_blocks
        else:
            free, total = torch.cuda.mem_get_info(self.device)
            if options.budget_gib:
                used = total - free
                room = int(options.budget_gib * GIB) - used
            else:
                room = int(free * options.kv_fraction)
            per_page = max(1, layout.bytes_per_token(itemsize) * options.block_size)
            num_pages = room // per_page
            if num_pages < 1:
                raise RuntimeError(f"no memory left for the cache pool ({room} bytes after the weights)")
        n_pages = [int(num_pages)] * len(layout.groups)
        max_step = options.max_step_tokens or (options.chunk_size * options.max_prefills_per_step + options.max_batch_size)
        self.cache = CacheManager(layout, options.block_size, n_pages, max_requests=options.max_batch_size)
        self.pools = DevicePools(layout, options.block_size, n_pages, options.max_batch_size, self.dtype,
                                 self.device, poison=options.poison_freed_pages)
        self.runner = ModelRunner(model, self.cache, self.pools, max_step_tokens=max_step,
                                  cuda_graphs=options.cuda_graphs, batch_invariant=options.batch_invariant,
                                  pad_decodes=options.pad_decodes, tune_products=options.tune_products)
        self.scheduler = Scheduler(self.cache, SchedulerConfig(
            max_batch_size=options.max_batch_size, prefill_chunk_size=options.chunk_size,
            max_prefills_per_step=options.max_prefills_per_step, max_step_tokens=max_step,
            reserve_pages=options.reserve_blocks, eos_token_id=options.eos_token_id,
            max_model_len=max_len, overcommit=options.overcommit))
        self.sampler = Sampler(self.device)
        self._next_id = 0
        self._requests: dict[str, Request] = {}
        self._in_flight: _Launched | None = None   # a step that runs on the device and has not been collected
        self.lookahead_steps = 0
        self.d2h_bytes_last = 0

    # --- construction -------------------------------------------------------------------------------

    @classmethod
    def from_pretrained(cls, folder: str | Path, options: EngineOptions | None = None, **overrides) -> "Engine":
        """Build from a folder with ``config.json`` and ``model.safetensors``."""
        options = _with(options, overrides)
        device, dtype = require_cuda(options.device), resolve_dtype(options.dtype)
        arch, config = read_model_folder(folder)
        plan = arch.make_plan(config)
        with torch.cuda.device(device):
            model = DecoderModel(plan, dtype, device)
            tensors = load_safetensors(folder, model.weight_specs(), dtype, device,
                                       plan.name_prefixes, plan.ignored_prefixes)
            model.load_weights(tensors)
            del tensors
            return cls(model, config, options)

    @classmethod
    def from_config(cls, raw_config: dict | str | Path, weights_seed: int = 0, std: float = 0.02,
                    options: EngineOptions | None = None, **overrides) -> "Engine":
        """Build with seeded random weights straight in device memory (no model folder)."""
        options = _with(options, overrides)
        device, dtype = require_cuda(options.device), resolve_dtype(options.dtype)
        if not isinstance(raw_config, dict):
            raw_config = json.loads(Path(raw_config).read_text())
        arch = architecture_of(raw_config)
        config = arch.read_config(raw_config, "config")
        plan = arch.make_plan(config)
        with torch.cuda.device(device):
            model = DecoderModel(plan, dtype, device)
            model.load_weights(random_tensors(model.weight_specs(), weights_seed, std, compute_dtype=dtype,
                                              device=device))
            return cls(model, config, options)

    # --- requests -----------------------------------------------------------------------------------

    def add_request(self, prompt_token_ids: list[int] | None = None, sampling: SamplingParams | None = None,
                    prompt_embeds: torch.Tensor | None = None, request_id: str | None = None) -> str:
        """Queue a prompt given as token ids, or as embedding rows ``[prompt_len, hidden]``."""
        sampling = sampling or SamplingParams()
        if prompt_embeds is not None:
            if prompt_embeds.dim() == 3 and prompt_embeds.shape[0] == 1:
                prompt_embeds = prompt_embeds[0]   # the reference's (1, P, H) layout
            if prompt_embeds.dim() != 2 or prompt_embeds.shape[1] != self.model.hidden_size:
                raise ValueError(f"prompt_embeds must be [prompt_len, {self.model.hidden_size}]")
            if prompt_token_ids is None:
                prompt_token_ids = [0] * prompt_embeds.shape[0]
            if len(prompt_token_ids) != prompt_embeds.shape[0]:
                raise ValueError("prompt_token_ids and prompt_embeds disagree in length")
            prompt_embeds = prompt_embeds.to(device=self.device, dtype=self.dtype)
        if prompt_token_ids is None:
            raise ValueError("a request needs prompt_token_ids or prompt_embeds")
        ids = [int(t) for t in prompt_token_ids]
        if prompt_embeds is None and any(not 0 <= t < self.model.vocab_size for t in ids):
            raise ValueError(f"a prompt token id is outside [0, {self.model.vocab_size})")
        rid = request_id if request_id is not None else f"req-{self._next_id}"
        if rid in self._requests and not self._requests[rid].is_finished:
            raise ValueError(f"request id {rid!r} is in use")
        seed = sampling.seed if sampling.seed is not None else self.options.seed * 1000003 + self._next_id
        self._next_id += 1
        request = Request(rid, ids, sampling, prompt_embeds, seed=seed)
        self._requests[rid] = request
        self.scheduler.add_request(request)
        return rid

    def abort(self, request_id: str, reason: str = "aborted") -> bool:
        """Stop a request wherever it is (queued, in a prompt, decoding, or in a step that is on the
        device): its pages and slot are free at once; a token that a launched step still produces for
        it is dropped.  Returns False if it had already finished."""
        request = self._requests[request_id]
        if request.is_finished:
            return False
        self.scheduler.abort(request, reason)
        return True

    def request(self, request_id: str) -> Request:
        return self._requests[request_id]

    @property
    def has_work(self) -> bool:
        return self.scheduler.has_work or self._in_flight is not None

    # --- one iteration ------------------------------------------------------------------------------

    def _entries(self, batch: Batch, fed_rows: dict[str, int] | None = None) -> list[StepEntry]:
        entries = []
        for e in batch.entries:
            r = e.request
            want = [e.n_tokens - 1] if e.samples else []
            if fed_rows is not None:
                entries.append(StepEntry(r.request_id, fed_back=fed_rows[r.request_id], want=want))
            elif e.from_embeds:
                entries.append(StepEntry(r.request_id, embeds=r.prompt_embeds[e.start: e.start + e.n_tokens], want=want))
            else:
                entries.append(StepEntry(r.request_id, tokens=[r.token_at(i) for i in range(e.start, e.start + e.n_tokens)],
                                         want=want))
        return entries

    def _launch(self, batch: Batch, after: "_Launched | None" = None) -> "_Launched":
        """Put one batch on the device: the step, the sampling kernel and the copy of the ids to the
        host.  ``after``: the step before, not yet collected; the batch's tokens are its samples."""
        fed_rows = None
        if after is not None:
            fed_rows = {e.request.request_id: row for row, e in enumerate(after.sampled)}
            self.runner.feedback = self.sampler.device_tokens
        try:
            logits = self.runner.step(self._entries(batch, fed_rows))
        except OutOfPagesError:
            if after is None:
                self._fail(batch, "OutOfPagesError")
            raise       # launched ahead: nothing was changed, the scheduler decides after the step before
        except Exception as exc:
            # Every request of the batch fails and frees its pages; the engine stays usable
            # (edgerag/serve/engine.py:178-189).
            self._fail(batch, type(exc).__name__)
            raise
        sampled = [e for e in batch.entries if e.samples]
        pending = None
        if sampled:
            ahead = 0 if after is None else 1            # the token of `after` is not in num_generated yet
            pending = self.sampler.launch(
                logits, [e.request.sampling for e in sampled], [e.request.seed for e in sampled],
                [e.request.num_generated + ahead for e in sampled])
        return _Launched(batch, sampled, pending)

    def _fail(self, batch: Batch, why: str) -> None:
        """A step of this batch raised, or its results are not valid: its requests end with
        ``finish_reason`` "error: ..." and give back their pages and slots."""
        for e in batch.entries:
            if not e.request.is_finished:
                self.scheduler.abort(e.request, f"error: {why}")

    def _following(self, cur: "_Launched") -> Batch | None:
        """The batch that follows ``cur`` if nothing unforeseen happens in it, or None when the next
        decision needs ``cur``'s tokens or the scheduler's judgement: every request of ``cur``
        samples (so each decodes next), those that reach their length limit with ``cur``'s token
        drop out, nobody else runs or could be admitted, and the pages for one more token are free."""
        sched = self.scheduler
        if not cur.sampled or len(cur.sampled) != len(cur.batch.entries) or len(sched.running) != len(cur.sampled):
            return None
        going = [e for e in cur.sampled if e.request.num_generated + 1 < e.request.max_new_tokens
                 and not e.request.is_finished]
        if not going or (sched.waiting and len(going) < sched.config.max_batch_size):
            return None
        need = [0] * len(self.cache.pages)
        for e in going:
            for g, n in enumerate(self.cache.pages_to_grow(e.request.request_id, 1)):
                need[g] += n
        if any(n > f for n, f in zip(need, self.cache.free_pages())):
            return None
        return Batch(cur.batch.step + 1, [ScheduledEntry(e.request, e.start + e.n_tokens, 1, False, True) for e in going])

    def _collect(self, done: "_Launched") -> list[TokenEvent]:
        """Read a launched step's tokens and commit it.  Entries of requests that finished meanwhile
        (a stop token in the step before) are dropped."""
        new_tokens: dict[str, int] = {}
        if done.pending is not None:
            tokens = done.pending.read()
            new_tokens = {e.request.request_id: t for e, t in zip(done.sampled, tokens)}
            try:
                self.runner.raise_if_flagged()       # reading synchronised: the status copy is current
            except Exception as exc:
                # A kernel of this step (or of one launched after it) gave up: nothing of it is kept.
                # A step launched ahead holds the same requests; it is dropped with them.
                self._fail(done.batch, type(exc).__name__)
                self._in_flight = None
                raise
            self.d2h_bytes_last = 4 * len(tokens)
        live = [e for e in done.sampled if not e.request.is_finished]
        self.scheduler.update(done.batch, new_tokens)
        events = []
        for e in live:
            r = e.request
            events.append(TokenEvent(r.request_id, new_tokens[r.request_id], r.num_generated - 1,
                                     r.state == RequestState.FINISHED, r.finish_reason))
        return events

    def step(self) -> list[TokenEvent]:
        """One iteration: returns the tokens of the oldest step that is on the device, after having
        launched the step that follows it where that needs no decision (``lookahead``).  Without
        lookahead: schedule, run and sample one batch, and return its tokens."""
        cur, self._in_flight = self._in_flight, None
        if cur is None:
            batch = self.scheduler.schedule()
            if batch.is_empty:
                return []
            cur = self._launch(batch)
        failure = None
        if self.options.lookahead:
            follow = self._following(cur)
            if follow is not None:
                try:
                    self._in_flight = self._launch(follow, after=cur)
                    self.lookahead_steps += 1
                except OutOfPagesError:
                    pass        # nothing was changed; the scheduler decides after this step
                except Exception as exc:
                    # The step launched ahead failed and took its requests with it (``_launch``).  The
                    # step before it is still collected, so that the scheduler's books and the cache
                    # agree for every request that goes on; then the failure is reported.
                    failure = exc
        events = self._collect(cur)
        if failure is not None:
            raise failure
        return events

    def stream(self) -> "Iterator[TokenEvent]":
        """Run steps while there is work and yield every generated token as soon as the host has it
        (the reference's ``InferenceEngine.stream``, edgerag/serve/engine.py:256-281, without the
        thread: the caller's loop drives the engine).  Requests may be added while iterating."""
        while self.has_work:
            before = self.scheduler.step_index
            events = self.step()
            yield from events
            if not events and self.scheduler.step_index == before and not self.scheduler.running:
                return      # nothing could be scheduled: what is left waits for pages that never come

    def generate(self, prompts: list[list[int]] | None = None, sampling: SamplingParams | list[SamplingParams] | None = None,
                 prompt_embeds: list[torch.Tensor | None] | None = None) -> list[list[int]]:
        """Generate for every prompt (token ids, or embeddings where ``prompt_embeds[i]`` is given)
        and return the new token ids of each, in the order of the prompts."""
        n = len(prompts) if prompts is not None else len(prompt_embeds or [])
        params = sampling if isinstance(sampling, list) else [sampling or SamplingParams()] * n
        ids = []
        for i in range(n):
            emb = prompt_embeds[i] if prompt_embeds is not None else None
            ids.append(self.add_request(prompts[i] if prompts is not None else None, params[i], emb))
        while self.has_work:
            before = self.scheduler.step_index
            self.step()
            if self.scheduler.step_index == before and not self.scheduler.running:
                break  # nothing could be scheduled: what is left waits for pages that never come
        out = []
        for rid in ids:
            r = self._requests[rid]
            if r.state == RequestState.REJECTED:
                raise RuntimeError(f"request {rid} was rejected: {r.finish_reason}")
            out.append(list(r.generated_token_ids))
        return out

    def stats(self) -> dict[str, Any]:
        return {"scheduler": self.scheduler.to_dict(), "cache": self.cache.to_dict(),
                "pool_bytes": self.pools.nbytes(), "workspace_bytes": self.runner.workspace.nbytes()}


def _with(options: EngineOptions | None, overrides: dict) -> EngineOptions:
    options = options or EngineOptions()
    if overrides:
        unknown = set(overrides) - set(options.__dataclass_fields__)
        if unknown:
            raise TypeError(f"unknown engine options: {sorted(unknown)}")
        options = EngineOptions(**{**options.__dict__, **overrides})
    return options
