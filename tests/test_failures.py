"""The failure path, with every fault injected on the host: a part whose ``forward`` raises, a code
written into the kernels' status word, steps that the step function must refuse.  The reference
fails every request of a batch whose forward raises, frees their blocks and keeps serving
(edgerag/serve/engine.py:178-189, tests/test_engine.py:186-219); the same is asked here of a step
that runs alone and of one that was launched ahead of the step before it.  No kernel is made to
fault, trap or wait in vain."""

from __future__ import annotations

import json

import pytest
import torch

import helpers
import plain_llama as plain

pytestmark = pytest.mark.gpu


class Boom(RuntimeError):
    pass


def register_faulty():
    """An architecture equal to the Llama decoder except that the feed-forward of layer 0 raises on a
    chosen call (one call per step).  Defined here; nothing of the framework changes."""
    from edgerag_b200.config import DecoderConfig, register_architecture
    from edgerag_b200.models.llama import llama_plan
    from edgerag_b200.parts.base import register_part
    from edgerag_b200.parts.swiglu import SwiGLU

    @register_part("ffn", "swiglu_raising")
    class RaisingSwiGLU(SwiGLU):
        graph_safe = False      # steps run eagerly, so that a call is a step
        calls = 0
        fail_at = -1

        def forward(self, x, ctx):
            cls = RaisingSwiGLU
            cls.calls += 1
            if cls.calls == cls.fail_at:
                raise Boom(f"injected failure in call {cls.calls}")
            return super().forward(x, ctx)

    def make_plan(cfg):
        plan = llama_plan(cfg)
        plan.layers[0].ffn.kind = "swiglu_raising"
        return plan

    register_architecture("FaultyLlamaForCausalLM", DecoderConfig.from_dict, make_plan)
    return RaisingSwiGLU


def faulty_folder(tmp_path, model_folders):
    """Tiny B's tensors under the faulty architecture's name."""
    src = model_folders("b", "float32", std=0.2)
    dst = tmp_path / "faulty"
    dst.mkdir()
    raw = json.loads((src / "config.json").read_text())
    raw["architectures"] = ["FaultyLlamaForCausalLM"]
    (dst / "config.json").write_text(json.dumps(raw))
    (dst / "model.safetensors").symlink_to(src / "model.safetensors")
    return src, dst


@pytest.mark.parametrize("lookahead", [False, True])
def test_a_raising_part_fails_its_batch_and_the_engine_goes_on(lookahead, tmp_path, model_folders):
    from edgerag_b200 import Engine, SamplingParams

    part = register_faulty()
    src, folder = faulty_folder(tmp_path, model_folders)
    cfg = plain.read_config(src)
    prompts = [helpers.random_sequence(cfg["vocab"], n, 70 + n) for n in (9, 14, 6)]
    params = [SamplingParams(max_new_tokens=n) for n in (12, 2, 12)]     # the second request is done before the fault
    options = dict(dtype="float32", block_size=8, num_blocks=24, chunk_size=16, max_batch_size=3,
                   max_prefills_per_step=3, lookahead=lookahead, poison_freed_pages=True)
    part.calls, part.fail_at = 0, -1
    want = Engine.from_pretrained(folder, **options).generate(prompts, params)

    engine = Engine.from_pretrained(folder, **options)
    # call 1 runs the three prompts, calls 2.. are decode steps; with lookahead, call 5 is a step that
    # is launched before the tokens of call 4 have been read
    part.calls, part.fail_at = 0, 5
    ids = [engine.add_request(p, s) for p, s in zip(prompts, params)]
    with pytest.raises(Boom):
        while engine.has_work:
            engine.step()
    part.fail_at = -1
    if lookahead:
        assert engine.lookahead_steps >= 1
    failed_a, done, failed_b = (engine.request(i) for i in ids)
    assert done.finish_reason == "length" and list(done.generated_token_ids) == want[1]
    for r, full in ((failed_a, want[0]), (failed_b, want[2])):
        assert r.is_finished and r.finish_reason == "error: Boom"
        # what it generated before the fault is what the run without a fault generated
        assert 0 < len(r.generated_token_ids) < 12 and list(r.generated_token_ids) == full[: len(r.generated_token_ids)]
    # pages and slots are back, nothing is in flight, the books agree
    engine.cache.check_invariants()
    assert engine.cache.free_pages() == [24] and engine.cache.slots.num_free == 3
    assert not engine.has_work and not engine.scheduler.running and engine._in_flight is None
    # and the same engine serves the same prompts as if nothing had happened
    assert engine.generate(prompts, params) == want
    engine.cache.check_invariants()
    assert engine.cache.free_pages() == [24]


@pytest.mark.parametrize("lookahead", [False, True])
def test_a_flagged_status_word_becomes_an_error_and_is_cleared(lookahead, model_folders):
    """What a kernel that gave up waiting leaves behind is a code in the status word.  Written there by
    the host, it must fail the step that was running, name the kind of fault, and leave the engine usable."""
    from edgerag_b200 import Engine, SamplingParams
    from edgerag_b200.engine.step import StepError

    folder = model_folders("b", "float32", std=0.2)
    cfg = plain.read_config(folder)
    prompts = [helpers.random_sequence(cfg["vocab"], n, 80 + n) for n in (11, 5)]
    options = dict(dtype="float32", block_size=8, num_blocks=16, chunk_size=16, max_batch_size=2,
                   max_prefills_per_step=2, lookahead=lookahead)
    want = Engine.from_pretrained(folder, **options).generate(prompts, SamplingParams(max_new_tokens=6))
    engine = Engine.from_pretrained(folder, **options)
    for code, needle in ((1000007, "attention kernel gave up"), (2000001, "attention kernel gave up"), (3, "flagged token 2")):
        ids = [engine.add_request(p, SamplingParams(max_new_tokens=6)) for p in prompts]
        engine.step()
        engine.step()
        engine.runner.status.fill_(code)
        with pytest.raises(StepError, match=needle):
            for _ in range(4):          # the code reaches the host with the next step's results
                engine.step()
        assert int(engine.runner.status) == 0
        for i in ids:
            assert engine.request(i).finish_reason == "error: StepError"
        engine.cache.check_invariants()
        assert engine.cache.free_pages() == [16] and engine.cache.slots.num_free == 2 and not engine.has_work
        assert engine.generate(prompts, SamplingParams(max_new_tokens=6)) == want


def test_refused_steps_leave_the_cache_untouched(model_folders):
    from edgerag_b200 import Engine
    from edgerag_b200.cache.manager import OutOfPagesError
    from edgerag_b200.engine.step import StepEntry, StepError

    folder = model_folders("a", "float32")
    cfg = plain.read_config(folder)
    engine = Engine.from_pretrained(folder, dtype="float32", block_size=16, num_blocks=4, max_batch_size=3,
                                    max_step_tokens=64, cuda_graphs=False)
    runner, cache = engine.runner, engine.cache
    runner.admit("a"), runner.admit("b")
    first = runner.step([StepEntry("a", tokens=[1, 2, 3], want=[2])]).clone()

    def books():
        return (cache.free_pages(), {r: (cache.requests[r].num_tokens, cache.held_pages(r)) for r in cache.requests})

    before = books()
    hidden = cfg["hidden"]
    refused = [
        ([], "at least one entry"),
        ([StepEntry("nobody", tokens=[1])], "not admitted"),
        ([StepEntry("a", tokens=[1]), StepEntry("a", tokens=[2])], "twice"),
        ([StepEntry("a", tokens=[cfg["vocab"]])], "outside"),
        ([StepEntry("a", tokens=[-1])], "outside"),
        ([StepEntry("a", tokens=[1, 2], want=[2])], "wanted place"),
        ([StepEntry("a", tokens=[])], "at least one token"),
        ([StepEntry("a", tokens=[1], embeds=torch.zeros(1, hidden))], "exactly one"),
        ([StepEntry("a", embeds=torch.zeros(2, hidden + 1))], "embeds must be"),
        ([StepEntry("a", fed_back=0)], "fed-back"),
        ([StepEntry("a", tokens=[1] * 30), StepEntry("b", tokens=[1] * 35)], "exceed the step limit"),
    ]
    for entries, needle in refused:
        with pytest.raises(StepError, match=needle):
            runner.step(entries)
        assert books() == before, needle
    # a step that needs more pages than are free changes nothing either: 4 pages of 16, "a" holds one
    with pytest.raises(OutOfPagesError):
        runner.step([StepEntry("a", tokens=[1] * 20), StepEntry("b", tokens=[2] * 36)])
    assert books() == before
    cache.check_invariants()
    # and the requests go on as if the refused steps had never been asked for
    again = Engine.from_pretrained(folder, dtype="float32", block_size=16, num_blocks=4, max_batch_size=3, cuda_graphs=False)
    again.runner.admit("a")
    assert torch.equal(again.runner.step([StepEntry("a", tokens=[1, 2, 3], want=[2])]), first)
    got = runner.step([StepEntry("a", tokens=[4, 5], want=[1])])
    want = again.runner.step([StepEntry("a", tokens=[4, 5], want=[1])])
    assert torch.equal(got, want)
