"""Generation through the Python entry point and the command line, against the plain implementation."""

from __future__ import annotations

import json
import subprocess
import sys

import pytest
import torch

import helpers
import plain_llama as plain

pytestmark = pytest.mark.gpu


def margins_ok(weights, cfg, prompt, tokens, min_margin):
    """Positions whose top-2 margin in the plain logits exceeds ``min_margin`` must agree
    (the reference's rule for 16-bit runs, tests/test_equivalence.py:260-324)."""
    seq = list(prompt)
    for t in tokens:
        logits = plain.forward(weights, cfg, seq)[-1]
        top = torch.topk(logits, 2).values
        if float(top[0] - top[1]) > min_margin:
            assert t == int(logits.argmax()), (len(seq) - len(prompt), t, int(logits.argmax()))
            seq.append(t)
        else:
            return   # a near-tie: the two runs may part ways from here on
    return


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b"])
def test_greedy_generation_matches_plain(which, dtype, model_folders):
    from edgerag_b200 import Engine, SamplingParams

    folder = model_folders(which, dtype, std=0.2)     # larger weights: decisive logits
    cfg, weights = plain.read_config(folder), plain.read_weights(folder)
    prompts = [helpers.random_sequence(cfg["vocab"], n, 40 + n) for n in ((7, 33) if which == "a" else (5, 40, 77))]
    engine = Engine.from_pretrained(folder, dtype=dtype, block_size=16 if which == "a" else 8, num_blocks=64,
                                    chunk_size=16, max_batch_size=3, poison_freed_pages=True)
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=16))
    assert engine.cache.free_pages() == [64] and not engine.has_work
    for prompt, out in zip(prompts, outs):
        assert len(out) == 16
        if dtype == "float32":
            assert out == plain.greedy_generate(weights, cfg, prompt, 16)
        else:
            margins_ok(weights, cfg, prompt, out, min_margin=0.05 * float(plain.forward(weights, cfg, prompt)[-1].abs().max()))
    # chunk size and batch composition do not change the tokens (tests/test_executor.py:120-191)
    engine2 = Engine.from_pretrained(folder, dtype=dtype, block_size=4, num_blocks=200, chunk_size=5, max_batch_size=1)
    if dtype == "float32":
        assert engine2.generate(prompts, SamplingParams(max_new_tokens=16)) == outs


@pytest.mark.parametrize("tag", ["a", "b"])
def test_tokens_of_the_reference_scheduler_and_executor(tag, tmp_path):
    """The committed greedy tokens of the reference's own ``Scheduler`` + ``ModelExecutor`` serving the
    golden prompts together with prompt portions of 4, 8 and 64 tokens (tests/golden/make_golden.py;
    edgerag tests/test_executor.py:120-191): this engine, with the same portion sizes, generates them."""
    from pathlib import Path

    from safetensors.torch import load_file

    from edgerag_b200 import Engine, SamplingParams

    raw, seed, std, n_new = {"a": (plain.TINY_A, 0, 0.05, 16), "b": (plain.TINY_B, 1, 0.08, 8)}[tag]
    folder = plain.write_model_folder(tmp_path / tag, raw, seed, std=std)
    golden = load_file(str(Path(__file__).resolve().parent / "golden" / f"golden_tiny_{tag}.safetensors"))
    n_prompts = sum(1 for key in golden if key.startswith("prompt_"))
    prompts = [golden[f"prompt_{i}"].tolist() for i in range(n_prompts)]
    for chunk in (4, 8, 64):
        engine = Engine.from_pretrained(folder, dtype="float32", block_size=8 if tag == "b" else 16, num_blocks=64,
                                        chunk_size=chunk, max_batch_size=n_prompts, max_prefills_per_step=1,
                                        poison_freed_pages=True)
        got = engine.generate(prompts, SamplingParams(max_new_tokens=n_new))
        assert got == [golden[f"served_chunk{chunk}_{i}"].tolist() for i in range(n_prompts)], chunk
        assert engine.cache.free_pages() == [64]


def test_cuda_graph_decode_equals_eager_decode(model_folders):
    """Decode-only steps replay a captured CUDA graph; the tokens and logits are those of the eager path."""
    from edgerag_b200 import Engine, SamplingParams
    from edgerag_b200.engine.step import StepEntry

    folder = model_folders("b", "bfloat16", std=0.2)
    cfg = plain.read_config(folder)
    prompts = [helpers.random_sequence(cfg["vocab"], n, 60 + n) for n in (9, 30, 17)]
    outs = {}
    for graphs in (False, True):
        engine = Engine.from_pretrained(folder, dtype="bfloat16", block_size=8, num_blocks=64, chunk_size=16,
                                        max_batch_size=3, max_prefills_per_step=3, cuda_graphs=graphs)
        outs[graphs] = engine.generate(prompts, SamplingParams(max_new_tokens=24))
        assert (engine.runner.graph_replays > 10) == graphs
    assert outs[True] == outs[False]
    # logits of a replayed step equal those of the same step run eagerly, bit for bit
    rows = {}
    for graphs in (False, True):
        engine = Engine.from_pretrained(folder, dtype="bfloat16", block_size=8, num_blocks=64, cuda_graphs=graphs)
        r = engine.runner
        r.admit("x"), r.admit("y")
        r.step([StepEntry("x", tokens=prompts[0]), StepEntry("y", tokens=prompts[1])])
        got = []
        for i in range(12):   # crosses a page boundary and a page-count bucket on the way
            got.append(r.step([StepEntry("x", tokens=[i + 1], want=[0]), StepEntry("y", tokens=[i + 2], want=[0])]).clone())
        rows[graphs] = torch.stack(got)
        assert (r.graph_replays > 0) == graphs
    assert torch.equal(rows[True], rows[False])
    # steps that mix a portion of a prompt with single tokens are captured too, once their layout repeats
    rows = {}
    for graphs in (False, True):
        engine = Engine.from_pretrained(folder, dtype="bfloat16", block_size=8, num_blocks=200, max_batch_size=8,
                                        cuda_graphs=graphs)
        r = engine.runner
        r.admit("x"), r.admit("y")
        r.step([StepEntry("x", tokens=prompts[0]), StepEntry("y", tokens=prompts[1])])
        got = []
        for i in range(10):           # the same layout again and again: a 16-token portion of a new request beside two single tokens
            r.admit(f"p{i}")
            out = r.step([StepEntry(f"p{i}", tokens=prompts[2][:16], want=[3, 15]), StepEntry("x", tokens=[i + 1], want=[0]),
                          StepEntry("y", tokens=[i + 2], want=[0])])
            got.append(out.clone())
            r.release(f"p{i}")
        rows[graphs] = torch.stack(got)
        assert (r.graph_replays >= 4) == graphs
    assert torch.equal(rows[True], rows[False])


def test_prompt_embeds_temperature_and_eos(model_folders):
    from edgerag_b200 import Engine, SamplingParams
    from edgerag_b200.ops.kernels import uniform_from_state
    from edgerag_b200.sampling.params import rng_state

    folder = model_folders("b", "float32", std=0.2)
    cfg, weights = plain.read_config(folder), plain.read_weights(folder)
    engine = Engine.from_pretrained(folder, dtype="float32", block_size=8, num_blocks=64, chunk_size=16, max_batch_size=4)
    prompt = helpers.random_sequence(cfg["vocab"], 20, 9)
    rows = plain.embed(weights, torch.tensor(prompt))
    by_ids, by_rows = engine.generate([prompt, None], SamplingParams(max_new_tokens=8), prompt_embeds=[None, rows])
    assert by_ids == by_rows == plain.greedy_generate(weights, cfg, prompt, 8)
    # N(0, 1) rows that are no token's embedding, with temperature 0.7 and a seed: every draw is where the
    # plain distribution and the request's own uniform put it, whatever else runs beside it
    emb = torch.randn((20, cfg["hidden"]), generator=torch.Generator().manual_seed(1))
    params = SamplingParams(temperature=0.7, seed=1, max_new_tokens=6)
    alone = engine.generate(None, params, prompt_embeds=[emb])[0]
    mixed = engine.generate([prompt, None, prompt[:5]], [SamplingParams(max_new_tokens=9), params, SamplingParams(max_new_tokens=3)],
                            prompt_embeds=[None, emb, None])
    assert mixed[1] == alone and mixed[0][:8] == by_ids
    h = emb
    for i, token in enumerate(alone):
        logits = plain.forward(weights, cfg, embeds=h)[-1]
        cdf = torch.cumsum(plain.temperature_probs(logits, 0.7), 0)
        u = uniform_from_state(rng_state(1, i))
        lo = float(cdf[token - 1]) if token else 0.0
        assert lo - 1e-4 <= u < float(cdf[token]) + 1e-4
        h = torch.cat([h, plain.embed(weights, torch.tensor([token]))])
    # an end-of-sequence id stops a request early and frees its pages
    first = by_ids[2]
    stopper = Engine.from_pretrained(folder, dtype="float32", block_size=8, num_blocks=64, eos_token_id=first)
    out = stopper.generate([prompt], SamplingParams(max_new_tokens=8))[0]
    assert out == by_ids[:3] and stopper.request("req-0").finish_reason == "stop"
    assert stopper.cache.free_pages() == [64]


def test_preemption_recomputes_to_the_same_tokens(model_folders):
    """With admission by current size and a pool too small for both requests, the newer one is
    evicted, recomputed later, and still produces the tokens it produces alone."""
    from edgerag_b200 import Engine, SamplingParams

    folder = model_folders("a", "float32", std=0.2)
    cfg = plain.read_config(folder)
    prompts = [helpers.random_sequence(cfg["vocab"], 30, 1), helpers.random_sequence(cfg["vocab"], 30, 2)]
    roomy = Engine.from_pretrained(folder, dtype="float32", block_size=16, num_blocks=32)
    want = roomy.generate(prompts, SamplingParams(max_new_tokens=40))
    tight = Engine.from_pretrained(folder, dtype="float32", block_size=16, num_blocks=7, overcommit=True,
                                   max_prefills_per_step=2, poison_freed_pages=True)
    got = tight.generate(prompts, SamplingParams(max_new_tokens=40))
    assert tight.scheduler.stats.preempted >= 1 and got == want
    assert tight.cache.free_pages() == [7]


def test_preemption_of_an_embedded_prompt_in_bfloat16(model_folders):
    """The same in bfloat16 with the evicted request given as ``prompt_embeds``: when it is readmitted,
    its embedded prompt is fed as rows again and its generated tokens as ids.  Recomputing in portions
    rounds differently from decoding token by token, so the tokens must equal the roomy run's up to the
    first place where the plain model's top-2 margin is not clear."""
    from edgerag_b200 import Engine, SamplingParams

    folder = model_folders("a", "bfloat16", std=0.2)
    cfg, weights = plain.read_config(folder), plain.read_weights(folder)
    ids = helpers.random_sequence(cfg["vocab"], 30, 1)
    rows = torch.randn((30, cfg["hidden"]), generator=torch.Generator().manual_seed(4)).to(torch.bfloat16)
    new = 40
    roomy = Engine.from_pretrained(folder, dtype="bfloat16", block_size=16, num_blocks=32)
    want = roomy.generate([ids, None], SamplingParams(max_new_tokens=new), prompt_embeds=[None, rows])
    tight = Engine.from_pretrained(folder, dtype="bfloat16", block_size=16, num_blocks=7, overcommit=True,
                                   max_prefills_per_step=2, poison_freed_pages=True)
    got = tight.generate([ids, None], SamplingParams(max_new_tokens=new), prompt_embeds=[None, rows])
    assert tight.scheduler.stats.preempted >= 1 and tight.request("req-1").preemptions >= 1
    assert tight.cache.free_pages() == [7] and [len(g) for g in got] == [new, new]
    heads = [plain.embed(weights, torch.tensor(ids)), rows.float()]
    agreed = 0
    for head, g, w in zip(heads, got, want):
        if g == w:
            agreed += new
            continue
        first = next(i for i in range(new) if g[i] != w[i])
        agreed += first
        embeds = torch.cat([head, plain.embed(weights, torch.tensor(w[:first]))]) if first else head
        logits = plain.forward(weights, cfg, embeds=embeds)[-1]
        top = torch.topk(logits, 2).values
        assert float(top[0] - top[1]) <= 0.05 * float(logits.abs().max()), (first, g[first], w[first])
    assert agreed >= new          # not vacuous: at least one request's worth of tokens agreed


def test_command_line(model_folders, tmp_path):
    folder = model_folders("a", "float32", std=0.2)
    cfg, weights = plain.read_config(folder), plain.read_weights(folder)
    prompt = helpers.random_sequence(cfg["vocab"], 12, 3)
    cmd = [sys.executable, "-m", "edgerag_b200", "--model", str(folder), "--dtype", "fp32", "--num-blocks", "32",
           "--chunk-size", "8", "--max-new-tokens", "6", "--prompt-ids", ",".join(map(str, prompt)), "--json"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=str(helpers.ROOT))
    assert proc.returncode == 0, proc.stderr[-3000:]
    out = json.loads(proc.stdout.strip().splitlines()[-1])
    assert out["outputs"][0]["token_ids"] == plain.greedy_generate(weights, cfg, prompt, 6)
    # random-weights mode: writes a folder and generates from it
    conf = tmp_path / "config.json"
    conf.write_text(json.dumps(plain.TINY_A))
    cmd = [sys.executable, "-m", "edgerag_b200", "--random-weights", "3", "--config", str(conf), "--save-model",
           str(tmp_path / "rw"), "--dtype", "bf16", "--num-blocks", "16", "--max-new-tokens", "4", "--prompt-ids", "1,2,3", "--json"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=str(helpers.ROOT))
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert (tmp_path / "rw" / "model.safetensors").is_file()
    assert len(json.loads(proc.stdout.strip().splitlines()[-1])["outputs"][0]["token_ids"]) == 4


def test_many_requests_through_a_small_pool_equal_each_alone(model_folders):
    """Continuous batching under pressure: a dozen requests of assorted lengths, a pool that holds
    about three of them, short portions, several prompts per step.  Every request must produce the
    tokens it produces alone (edgerag tests/test_executor.py:164-191), and every page must come back."""
    from edgerag_b200 import Engine, SamplingParams

    folder = model_folders("b", "float32", std=0.2)
    cfg = plain.read_config(folder)
    lens = [5, 61, 17, 40, 9, 77, 23, 3, 50, 31, 12, 66]
    news = [9, 4, 17, 6, 30, 5, 12, 25, 7, 11, 19, 3]
    prompts = [helpers.random_sequence(cfg["vocab"], n, 300 + n) for n in lens]
    solo = Engine.from_pretrained(folder, dtype="float32", block_size=8, num_blocks=64, chunk_size=512, max_batch_size=1)
    want = [solo.generate([p], SamplingParams(max_new_tokens=n))[0] for p, n in zip(prompts, news)]
    busy = Engine.from_pretrained(folder, dtype="float32", block_size=8, num_blocks=30, chunk_size=11, max_batch_size=5,
                                  max_prefills_per_step=2, poison_freed_pages=True)
    got = busy.generate(prompts, [SamplingParams(max_new_tokens=n) for n in news])
    assert got == want
    stats = busy.scheduler.stats
    assert stats.finished == len(prompts) and stats.admission_blocked > 0 and stats.preempted == 0
    assert busy.cache.free_pages() == [30] and busy.cache.slots.num_free == 5
    busy.cache.check_invariants()


def test_lookahead_changes_no_token(model_folders):
    """With lookahead the engine launches the next decoding step before it has read this step's
    tokens (they are fed back on the device).  Greedy and seeded temperature requests of assorted
    lengths, a stop token that ends one request in the middle (so that a step launched ahead has to
    be dropped for it), a queue that waits for slots: every request produces what it produces
    without lookahead, the events come in the same order, and every page comes back."""
    from edgerag_b200 import Engine, SamplingParams

    folder = model_folders("a", "float32", std=0.2)
    cfg = plain.read_config(folder)
    prompts = [helpers.random_sequence(cfg["vocab"], n, 500 + n) for n in (12, 33, 5, 21, 40, 9)]
    params = [SamplingParams(max_new_tokens=n) for n in (20, 7, 31, 1, 12, 26)]
    params[1] = SamplingParams(max_new_tokens=18, temperature=0.8, seed=3)
    params[4] = SamplingParams(max_new_tokens=15, temperature=1.3, seed=9)
    probe = Engine.from_pretrained(folder, dtype="float32", block_size=8, num_blocks=64, max_batch_size=1, lookahead=False)
    eos = probe.generate([prompts[0]], SamplingParams(max_new_tokens=20))[0][9]      # request 0 stops at its tenth token at the latest
    runs = {}
    for ahead in (False, True):
        engine = Engine.from_pretrained(folder, dtype="float32", block_size=8, num_blocks=40, chunk_size=16, max_batch_size=4,
                                        max_prefills_per_step=2, eos_token_id=eos, lookahead=ahead, poison_freed_pages=True)
        for p, sp in zip(prompts, params):
            engine.add_request(p, sp)
        events = []
        while engine.has_work:
            events.extend((e.request_id, e.token_id, e.index, e.finished, e.finish_reason) for e in engine.step())
        runs[ahead] = (events, [engine.request(f"req-{i}").generated_token_ids for i in range(len(prompts))])
        assert (engine.lookahead_steps > 10) == ahead
        assert engine.cache.free_pages() == [40] and engine.cache.slots.num_free == 4
        engine.cache.check_invariants()
        assert engine.request("req-0").finish_reason == "stop" and len(runs[ahead][1][0]) <= 10
    assert runs[True][1] == runs[False][1]
    assert sorted(runs[True][0]) == sorted(runs[False][0])
    for rid in {e[0] for e in runs[True][0]}:         # each request's events in order, with and without
        assert [e for e in runs[True][0] if e[0] == rid] == [e for e in runs[False][0] if e[0] == rid]


def test_stream_yields_tokens_as_they_come(model_folders):
    """``Engine.stream`` yields every token with its request and index, in order per request, a request
    added half-way joins in, and the tokens are those of ``generate``."""
    from edgerag_b200 import Engine, SamplingParams

    folder = model_folders("a", "float32", std=0.2)
    cfg = plain.read_config(folder)
    prompts = [helpers.random_sequence(cfg["vocab"], n, 700 + n) for n in (11, 29, 6)]
    whole = Engine.from_pretrained(folder, dtype="float32", block_size=8, num_blocks=64, max_batch_size=4)
    want = whole.generate(prompts, SamplingParams(max_new_tokens=12))
    engine = Engine.from_pretrained(folder, dtype="float32", block_size=8, num_blocks=64, max_batch_size=4)
    ids = [engine.add_request(p, SamplingParams(max_new_tokens=12)) for p in prompts[:2]]
    got: dict[str, list[int]] = {}
    for n, ev in enumerate(engine.stream()):
        assert ev.index == len(got.setdefault(ev.request_id, []))
        got[ev.request_id].append(ev.token_id)
        assert ev.finished == (len(got[ev.request_id]) == 12)
        if n == 5:
            ids.append(engine.add_request(prompts[2], SamplingParams(max_new_tokens=12)))
    assert [got[i] for i in ids] == want and not engine.has_work


def test_abort_frees_at_once_and_disturbs_nobody(model_folders):
    """A request aborted while a step launched ahead still carries it: its pages and slot come back at
    once, its late token is dropped, the other request's tokens are what they are alone."""
    from edgerag_b200 import Engine, SamplingParams

    folder = model_folders("b", "float32", std=0.2)
    cfg = plain.read_config(folder)
    prompts = [helpers.random_sequence(cfg["vocab"], n, 800 + n) for n in (14, 23)]
    alone = Engine.from_pretrained(folder, dtype="float32", block_size=8, num_blocks=32, max_batch_size=1)
    want = alone.generate([prompts[1]], SamplingParams(max_new_tokens=20))[0]
    engine = Engine.from_pretrained(folder, dtype="float32", block_size=8, num_blocks=32, max_batch_size=2,
                                    max_prefills_per_step=2, poison_freed_pages=True)
    a = engine.add_request(prompts[0], SamplingParams(max_new_tokens=50))
    b = engine.add_request(prompts[1], SamplingParams(max_new_tokens=20))
    for _ in range(6):
        engine.step()
    assert engine.lookahead_steps > 0 and engine.abort(a) and not engine.abort(a)
    held_by_b = sum(engine.cache.held_pages(b))
    assert engine.cache.free_pages() == [32 - held_by_b] and engine.request(a).finish_reason == "aborted"
    n_a = len(engine.request(a).generated_token_ids)
    for ev in engine.stream():
        assert ev.request_id == b
    assert engine.request(b).generated_token_ids == want and len(engine.request(a).generated_token_ids) == n_a
    assert engine.cache.free_pages() == [32] and engine.cache.slots.num_free == 2


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_filler_rows_change_no_token_and_save_graphs(dtype, tmp_path):
    """Requests that finish at different times make the number of single-token rows fall from 5 to 1; with
    filler rows the steps are laid out for 8, 4, 2 and 1 rows, so fewer layouts are captured and more
    steps replayed, and the tokens are those of an engine without fillers.  Free pages hold NaN, which
    the fillers read (page 0 may be free) and which must reach nobody else."""
    import shutil

    from edgerag_b200 import Engine, SamplingParams

    folder = plain.write_model_folder(tmp_path, plain.TINY_A, seed=3, std=0.2, dtype=getattr(torch, dtype))
    try:
        prompts = [helpers.random_sequence(512, 20 + 9 * i, 40 + i) for i in range(5)]
        news = [6, 30, 14, 40, 22]
        outs, stats = {}, {}
        for fill in (False, True):
            engine = Engine.from_pretrained(folder, dtype=dtype, block_size=16, num_blocks=40, max_batch_size=8, chunk_size=64,
                                            max_prefills_per_step=5, cuda_graphs=True, pad_decodes=fill, poison_freed_pages=True)
            # (two of the requests sample with a temperature: their draws depend on the request and the token's
            # index only, so the filler rows must not shift them either)
            ids = [engine.add_request(p, SamplingParams(max_new_tokens=n, temperature=0.8 if i % 2 else 0.0, seed=17 + i))
                   for i, (p, n) in enumerate(zip(prompts, news))]
            got = {i: [] for i in ids}
            for ev in engine.stream():
                got[ev.request_id].append(ev.token_id)
            outs[fill] = [got[i] for i in ids]
            stats[fill] = (len(engine.runner._graphs), engine.runner.graph_replays)
            assert engine.cache.free_pages() == [40]
        assert [len(o) for o in outs[True]] == news
        if dtype == "float32":
            assert outs[True] == outs[False]
        else:
            # bfloat16: the attention kernel's launch shape follows the number of rows, so the two engines may
            # round differently; each follows the plain model wherever its top-2 margin is clear
            cfg, weights = plain.read_config(folder), plain.read_weights(folder)
            checked = 0
            for fill in (False, True):
                for i, (prompt, out) in enumerate(zip(prompts, outs[fill])):
                    if i % 2:
                        continue        # (sampled: judged in float32 only, where the two engines must agree)
                    logits = plain.forward(weights, cfg, list(prompt) + out[:-1])[len(prompt) - 1:]
                    for got, row in zip(out, logits):
                        top = torch.topk(row, 2).values
                        if float(top[0] - top[1]) >= 0.05 * float(row.abs().max()):
                            assert got == int(row.argmax())
                            checked += 1
            assert checked >= sum(news[::2])
        assert stats[True][0] <= stats[False][0] and stats[True][1] >= stats[False][1], stats
        assert stats[True][1] > stats[False][1] or stats[True][0] < stats[False][0], stats
    finally:
        shutil.rmtree(tmp_path, ignore_errors=True)
