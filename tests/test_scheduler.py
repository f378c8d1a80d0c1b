"""The scheduler's decisions, against the real (tensor-free) cache manager and a stand-in runner."""

from __future__ import annotations

import random

import pytest

from edgerag_b200.cache.manager import CacheLayout, CacheManager, KVGroupSpec
from edgerag_b200.engine.request import Request, RequestState
from edgerag_b200.engine.scheduler import Batch, Scheduler, SchedulerConfig
from edgerag_b200.sampling.params import SamplingParams


def make(num_pages=32, page_size=4, slots=8, **cfg) -> tuple[Scheduler, CacheManager]:
    layout = CacheLayout(groups=[KVGroupSpec(2, 1, 16, 0)], placement=[(0, 0), (0, 1)])
    cache = CacheManager(layout, page_size, num_pages, max_requests=slots)
    return Scheduler(cache, SchedulerConfig(**cfg)), cache


def req(rid: str, prompt_len: int, new: int = 4) -> Request:
    return Request(rid, list(range(1, prompt_len + 1)), SamplingParams(max_new_tokens=new))


def run_step(s: Scheduler, cache: CacheManager, token=lambda r: 7) -> Batch:
    """What the engine does around a step, with the model replaced by a constant token."""
    batch = s.schedule()
    for e in batch.entries:
        cache.grow(e.request.request_id, e.n_tokens)
    for e in batch.entries:
        cache.advance(e.request.request_id, e.n_tokens)
    s.update(batch, {e.request.request_id: token(e.request) for e in batch.entries if e.samples})
    cache.check_invariants()
    return batch


def test_portions_then_decode_then_finish_frees():
    s, cache = make(prefill_chunk_size=8, max_batch_size=4)
    r = req("a", 19, new=3)
    assert s.add_request(r)
    b = run_step(s, cache)
    assert [(e.start, e.n_tokens, e.samples) for e in b.entries] == [(0, 8, False)]
    assert r.state is RequestState.PREFILLING and r.num_computed == 8 and not r.generated_token_ids
    run_step(s, cache)
    b = run_step(s, cache)                      # last portion: 3 tokens, yields the first new token
    assert [(e.start, e.n_tokens, e.samples) for e in b.entries] == [(16, 3, True)]
    assert r.generated_token_ids == [7] and r.state is RequestState.DECODING and r.first_token_step == 2
    b = run_step(s, cache)
    assert b.entries[0].is_decode and b.entries[0].start == 19
    run_step(s, cache)
    assert r.state is RequestState.FINISHED and r.finish_reason == "length" and r.generated_token_ids == [7, 7, 7]
    assert cache.free_pages() == [32] and not s.has_work and s.stats.finished == 1
    # the third token is sampled, never fed: the cache held prompt + 2 tokens
    assert s.stats.decode_tokens == 2 and s.stats.prefill_portions == 3


def test_eos_stops_and_reports_stop():
    s, cache = make(eos_token_id=5)
    r = req("a", 3, new=10)
    s.add_request(r)
    run_step(s, cache, token=lambda r: 9)
    run_step(s, cache, token=lambda r: 5)
    assert r.finish_reason == "stop" and r.generated_token_ids == [9, 5]


def test_a_step_launched_ahead_for_a_request_that_stopped_is_dropped():
    """The engine may launch the step that follows before it has read this step's tokens.  If a
    request turns out to have stopped on its stop token, the entry of the step launched ahead is
    skipped when that step is committed: no token appended, nothing counted, nothing freed twice."""
    from edgerag_b200.engine.scheduler import ScheduledEntry

    s, cache = make(prefill_chunk_size=8, max_batch_size=4, eos_token_id=9)
    a, b = req("a", 5, new=6), req("b", 3, new=6)
    s.add_request(a), s.add_request(b)
    run_step(s, cache)                        # a's prompt and its first token
    run_step(s, cache)                        # a decodes, b's prompt
    cur = s.schedule()                        # both decode
    assert [e.request.request_id for e in cur.entries] == ["a", "b"] and all(e.is_decode for e in cur.entries)
    for e in cur.entries:
        cache.grow(e.request.request_id, 1), cache.advance(e.request.request_id, 1)
    ahead = Batch(cur.step + 1, [ScheduledEntry(e.request, e.start + 1, 1, False, True) for e in cur.entries])
    for e in ahead.entries:                   # launched before cur's tokens are known
        cache.grow(e.request.request_id, 1), cache.advance(e.request.request_id, 1)
    done = s.update(cur, {"a": 9, "b": 7})    # a stops on its stop token
    assert done == [a] and a.finish_reason == "stop" and "a" not in cache.requests
    before = (list(a.generated_token_ids), s.stats.decode_tokens, s.stats.finished)
    s.update(ahead, {"a": 5, "b": 8})
    assert (list(a.generated_token_ids), s.stats.finished) == (before[0], before[2])
    assert s.stats.decode_tokens == before[1] + 1 and b.generated_token_ids[-2:] == [7, 8]
    cache.check_invariants()
    while s.has_work:
        run_step(s, cache)
    assert cache.free_pages() == [32]


def test_decodes_first_one_prefill_per_step_fifo_admission():
    s, cache = make(num_pages=64, prefill_chunk_size=4, max_batch_size=3, max_prefills_per_step=1)
    a, b, c, d = req("a", 2, 8), req("b", 9, 8), req("c", 3, 8), req("d", 3, 8)
    for r in (a, b, c, d):
        s.add_request(r)
    assert [e.request.request_id for e in run_step(s, cache).entries] == ["a"]          # one prefill per step
    assert [e.request.request_id for e in run_step(s, cache).entries] == ["a", "b"]     # decode first, then admit b
    batch = run_step(s, cache)
    assert [(e.request.request_id, e.n_tokens) for e in batch.entries] == [("a", 1), ("b", 4)]  # b mid-prompt blocks c
    run_step(s, cache)                                                                     # b's last portion (1 token)
    batch = run_step(s, cache)
    assert [e.request.request_id for e in batch.entries] == ["a", "b", "c"]               # now c is admitted
    batch = run_step(s, cache)
    assert [e.request.request_id for e in batch.entries] == ["a", "b", "c"]               # batch is full: d waits
    assert s.waiting[0] is d


def test_token_budget_cuts_the_portion():
    s, cache = make(num_pages=64, prefill_chunk_size=16, max_batch_size=4, max_step_tokens=6, max_prefills_per_step=2)
    a, b = req("a", 2, 20), req("b", 30, 2)
    s.add_request(a)
    run_step(s, cache)
    s.add_request(b)
    batch = run_step(s, cache)
    assert [(e.request.request_id, e.n_tokens) for e in batch.entries] == [("a", 1), ("b", 5)]
    assert batch.n_tokens == 6


def test_admission_budgets_the_final_size_and_commits_it():
    # 10 pages of 4 tokens.  a: 6 + 10 -> 4 pages; b: 8 + 12 -> 5 pages; c: 4 + 4 -> 2 pages.
    s, cache = make(num_pages=10, prefill_chunk_size=16, max_batch_size=4, max_prefills_per_step=4)
    a, b, c = req("a", 6, 10), req("b", 8, 12), req("c", 4, 4)
    for r in (a, b, c):
        s.add_request(r)
    batch = run_step(s, cache)
    # a and b are admitted (9 pages committed); c would need 2 of the 1 uncommitted page and waits,
    # although 6 pages are still physically free.
    assert [e.request.request_id for e in batch.entries] == ["a", "b"]
    assert cache.free_pages() == [6] and s.available_pages() == [1] and s.stats.admission_blocked == 1
    while a.state is not RequestState.FINISHED:
        run_step(s, cache)
    assert c.state is RequestState.WAITING
    run_step(s, cache)
    assert c.state is not RequestState.WAITING          # a's pages came back: c gets in at the next step
    while s.has_work:
        run_step(s, cache)
    assert cache.free_pages() == [10] and s.stats.preempted == 0


def test_requests_that_can_never_fit_are_rejected_at_once():
    s, cache = make(num_pages=4, page_size=4, max_model_len=64)
    big, long = req("big", 14, 4), req("long", 60, 8)
    assert not s.add_request(big) and big.state is RequestState.REJECTED and big.finish_reason == "exceeds_pool"
    assert not s.add_request(long) and long.finish_reason == "too_long"
    assert not s.add_request(Request("e", [], SamplingParams())) and s.stats.rejected == 3
    assert not s.has_work


def test_overcommit_preempts_newest_first_and_recomputes():
    s, cache = make(num_pages=6, page_size=4, prefill_chunk_size=8, max_batch_size=3, max_prefills_per_step=3,
                    overcommit=True)
    a, b = req("a", 7, 12), req("b", 7, 12)
    s.add_request(a)
    s.add_request(b)
    steps = 0
    while s.stats.preempted == 0:
        run_step(s, cache)
        steps += 1
        assert steps < 50
    # the newer request was evicted, keeps what it generated, and waits at the front of the queue
    assert s.waiting[0] is b and b.state is RequestState.WAITING and b.num_computed == 0 and b.preemptions == 1
    assert b.request_id not in cache.requests and a in s.running
    had = list(b.generated_token_ids)
    assert had
    while a.state is not RequestState.FINISHED:
        run_step(s, cache)
    batch = run_step(s, cache)
    e = next(e for e in batch.entries if e.request is b)
    assert e.start == 0 and e.n_tokens == min(8, b.prompt_len + len(had))   # recomputes prompt and generated tokens
    while s.has_work:
        run_step(s, cache)
    assert b.generated_token_ids[: len(had)] == had and len(b.generated_token_ids) == 12
    assert cache.free_pages() == [6]


def test_alone_and_out_of_pages_is_rejected_not_spun():
    s, cache = make(num_pages=3, page_size=4, overcommit=True, prefill_chunk_size=4)
    r = req("a", 6, 4)            # final size 10 tokens = 3 pages: passes the static check
    cache.admit("other")                 # someone outside the scheduler holds a page
    cache.grow("other", 4)
    s.add_request(r)
    for _ in range(6):
        run_step(s, cache)
    assert r.state is RequestState.REJECTED and r.finish_reason == "out_of_pages"
    cache.release("other")
    assert cache.free_pages() == [3]


def test_embedded_prompts_never_mix_rows_and_ids_in_one_portion():
    r = Request("e", [0] * 5, SamplingParams(max_new_tokens=4), prompt_embeds=object())
    r.generated_token_ids = [3, 4]
    assert r.next_portion(16) == (0, 5, True)       # stops at the end of the embedded prompt
    r.num_computed = 5
    assert r.next_portion(16) == (5, 2, False)
    assert r.token_at(5) == 3 and r.token_at(6) == 4


@pytest.mark.parametrize("seed", range(4))
def test_random_load_conserves_pages_and_finishes_everything(seed):
    rng = random.Random(seed)
    s, cache = make(num_pages=24, page_size=4, prefill_chunk_size=rng.choice([3, 8, 16]), max_batch_size=4,
                    max_prefills_per_step=rng.choice([1, 2]), overcommit=bool(seed % 2))
    made = []
    for step in range(400):
        if rng.random() < 0.3 and len(made) < 40:
            r = req(f"r{len(made)}", rng.randint(1, 30), rng.randint(1, 12))
            s.add_request(r)
            made.append(r)
        run_step(s, cache, token=lambda r: rng.randint(0, 9))
    while s.has_work:
        before = (s.step_index, len(s.finished))
        run_step(s, cache)
        assert (s.step_index, len(s.finished)) != before
    assert all(r.is_finished for r in made)
    ok = [r for r in made if r.state is RequestState.FINISHED]
    assert all(len(r.generated_token_ids) == r.max_new_tokens for r in ok) and len(ok) >= len(made) - 2
    assert cache.free_pages() == [24] and cache.slots.num_free == 8
