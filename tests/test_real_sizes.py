"""The layer sizes of the real SmolVLM decoders (two layers each, random weights), so that the
kernels which only take those shapes (tensor-core prefill attention and bulk-copy decode attention at
head size 64, the weight-streaming products, an odd vocabulary) are checked inside the engine and not
only alone: every cutting of a request against the plain implementation, in bfloat16 and in 32-bit."""

from __future__ import annotations

import pytest
import torch

import helpers
import plain_llama as plain

pytestmark = pytest.mark.gpu

SIZES = {
    # SmolVLM-2.2B decoder: 32 query and 32 kv heads of 64, odd vocabulary
    "2b": dict(hidden_size=2048, num_attention_heads=32, num_key_value_heads=32, head_dim=64, intermediate_size=8192,
               vocab_size=49155, rope_theta=273768.0),
    # SmolVLM-256M decoder: 9 query heads on 3 kv heads
    "256m": dict(hidden_size=576, num_attention_heads=9, num_key_value_heads=3, head_dim=64, intermediate_size=1536,
                 vocab_size=49280, rope_theta=100000.0),
    # SmolVLM-500M decoder: 15 query heads on 5 kv heads (one decode block serves all five)
    "500m": dict(hidden_size=960, num_attention_heads=15, num_key_value_heads=5, head_dim=64, intermediate_size=2560,
                 vocab_size=49280, rope_theta=100000.0),
}


def folder_for(tmp, which, dtype):
    raw = {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
           "max_position_embeddings": 8192, "hidden_act": "silu", **SIZES[which]}
    # larger weights than N(0, 0.02) so that attention is not near-uniform and logits are O(1)
    return plain.write_model_folder(tmp / f"{which}_{dtype}", raw, seed=3, std=0.04 if which == "2b" else 0.06,
                                    dtype=getattr(torch, dtype))


def add_cuttings(trace, vocab, prefix=""):
    """Every cutting of three sequences (333, 140 and 70 tokens), with request names under ``prefix``."""
    base = {"s0": helpers.random_sequence(vocab, 333, 1), "s1": helpers.random_sequence(vocab, 140, 2),
            "s2": helpers.random_sequence(vocab, 70, 3)}
    for tag in ("whole", "tail", "portions", "mixed"):
        for rid, seq in base.items():
            trace.sequences[f"{prefix}{tag}-{rid}"] = seq
    name = lambda tag, rid: f"{prefix}{tag}-{rid}"      # noqa: E731

    def want_last(n):      # logits of a few places per step keep the files small at a 49k vocabulary
        return sorted({0, n - 1, n // 2})

    for rid in base:
        n = trace.remaining(name("whole", rid))
        trace.add_step([(name("whole", rid), n, want_last(n))], end=[name("whole", rid)])
    tail = name("tail", "s0")
    n = trace.remaining(tail)
    trace.add_step([(tail, n - 32, want_last(n - 32))])
    for i in range(32):
        trace.add_step([(tail, 1, "all")], end=[tail] if i == 31 else [])
    sizes = (130, 2, 65, 3, 128, 5)
    i = 0
    por = name("portions", "s0")
    while trace.remaining(por):
        n = min(sizes[i % len(sizes)], trace.remaining(por))
        if trace.remaining(por) - n == 1:
            n += 1
        trace.add_step([(por, n, want_last(n))], end=[por] if trace.remaining(por) == n else [])
        i += 1
    # mixed: portions of one request beside single tokens of the others, pages reused afterwards
    m0, m1, m2 = (name("mixed", r) for r in ("s0", "s1", "s2"))
    trace.add_step([(m0, 200, [199]), (m1, 100, [99])])
    trace.add_step([(m0, 1, "all"), (m1, 39, [38]), (m2, 50, [49])])
    for _ in range(20):
        trace.add_step([(m0, 1, "all"), (m1, 1, "all") if trace.remaining(m1) else (m2, 1, "all")])
    trace.add_step([(m0, trace.remaining(m0), "last")], end=[m0, m1])
    trace.add_step([(m2, trace.remaining(m2), "last")], end=[m2])


def replay_and_compare(folder, dtype, trace, out_dir, label, extra=(), info=None):
    results = helpers.run_trace(folder, dtype, trace, out_dir, extra=("--poison-freed-pages", *extra), info=info)
    reference = helpers.plain_reference(folder, {k: v for k, v in trace.sequences.items()
                                                 if any(k == e[2] for e in trace.expect)})
    return results, helpers.compare(trace, results, reference, dtype, label=label)


@pytest.mark.parametrize("which,dtype", [("2b", "bfloat16"), ("2b", "float32"), ("256m", "bfloat16"), ("256m", "float32"),
                                         ("500m", "bfloat16")])
def test_cuttings_at_real_layer_sizes(which, dtype, tmp_path):
    import shutil

    folder = folder_for(tmp_path, which, dtype)
    cfg = plain.read_config(folder)
    trace = helpers.Trace()
    add_cuttings(trace, cfg["vocab"])
    try:
        _, stats = replay_and_compare(folder, dtype, trace, tmp_path / "out", f"{which} sizes")
        print(which, dtype, stats)
    finally:
        shutil.rmtree(tmp_path, ignore_errors=True)      # up to a gigabyte of weights and logits


@pytest.mark.parametrize("which,dtype", [("2b", "bfloat16"), ("500m", "bfloat16"), ("256m", "float32")])
def test_cuttings_replayed_from_cuda_graphs(which, dtype, tmp_path):
    """The same cuttings three times over in one process with CUDA graphs on, as serving runs: a layout is
    captured the second time it is seen and replayed from then on, so the third pass (and the decode
    steps of every pass) come out of graphs.  Same bands against the plain model; and a replayed step
    gives the bits of the step that was launched kernel by kernel.  (The two runs are two processes; both take
    the library's first proposal for every product, the engine's default: with ``tune_products`` each process
    would keep its own choice among the proposals, by timing them.)"""
    import re
    import shutil

    import numpy as np

    folder = folder_for(tmp_path, which, dtype)
    cfg = plain.read_config(folder)
    trace = helpers.Trace()
    for prefix in ("r0-", "r1-", "r2-"):
        add_cuttings(trace, cfg["vocab"], prefix)
    try:
        info = {}
        with_graphs, stats = replay_and_compare(folder, dtype, trace, tmp_path / "graphs", f"{which} sizes, graphs",
                                                extra=("--cuda-graphs",), info=info)
        found = re.search(r"cuda graphs: (\d+) captured, (\d+) steps replayed", info["stderr"])
        assert found, info["stderr"][-500:]
        n_steps = len(trace.steps)
        # the whole third pass and the decode steps of the first two are replays
        assert int(found.group(2)) >= n_steps // 3 + 60, (found.group(0), n_steps)
        print(which, dtype, stats, found.group(0))
        eager = helpers.run_trace(folder, dtype, trace, tmp_path / "eager", extra=("--poison-freed-pages",))
        for step in with_graphs:
            assert np.array_equal(with_graphs[step], eager[step]), f"step {step} differs between a graph and kernel launches"
    finally:
        shutil.rmtree(tmp_path, ignore_errors=True)


@pytest.mark.parametrize("which", ["2b", "500m"])
def test_generation_with_graphs_and_lookahead_at_real_layer_sizes(which, tmp_path):
    """The configuration that is timed (bfloat16, CUDA graphs, steps launched ahead, the head-size-64
    kernels) through ``Engine.generate``: prompts long enough that every decode step merges several
    key splits, freed pages poisoned.  Graphs and lookahead, on or off, change no token; the tokens
    are the plain model's wherever its top-2 margin is clear; a stop token that ends one request in
    the middle (a step launched ahead is dropped for it) changes nothing for the others."""
    import itertools
    import shutil

    from edgerag_b200 import Engine, SamplingParams
    from edgerag_b200.ops import kernels

    folder = folder_for(tmp_path, which, "bfloat16")
    try:
        cfg, weights = plain.read_config(folder), plain.read_weights(folder)
        lens, new = (700, 450, 90), 20
        prompts = [helpers.random_sequence(cfg["vocab"], n, 900 + n) for n in lens]
        options = dict(dtype="bfloat16", block_size=16, num_blocks=100, chunk_size=512, max_batch_size=3,
                       max_prefills_per_step=3, poison_freed_pages=True)
        bound, granule = kernels.context_bound(-(-lens[0] // 16))
        split = kernels.choose_decode_plan(3, cfg["n_kv"], bound * 16, 16, cfg["head_dim"], cfg["n_q"] != cfg["n_kv"], granule * 16)[0]
        assert lens[0] // split + 1 >= 3, f"splits of {split} keys: the longest request would have fewer than three"
        runs = {}
        for graphs, ahead in itertools.product((False, True), (False, True)):
            engine = Engine.from_pretrained(folder, cuda_graphs=graphs, lookahead=ahead, **options)
            runs[(graphs, ahead)] = engine.generate(prompts, SamplingParams(max_new_tokens=new))
            assert (engine.runner.graph_replays >= new - 8) == graphs and (engine.lookahead_steps >= new - 8) == ahead
            assert engine.cache.free_pages() == [100]
        base = runs[(False, False)]
        for key, outs in runs.items():
            assert outs == base, f"graphs={key[0]} lookahead={key[1]} changed a token"
        checked = 0
        for prompt, out in zip(prompts, base):
            # the plain model reads the engine's own tokens, so every place can be judged on its own:
            # where the plain top-2 margin is clear, the engine must have chosen the plain argmax
            logits = plain.forward(weights, cfg, prompt + out[:-1])[len(prompt) - 1:]
            floor = 0.05 * float(logits.abs().max())
            for i, token in enumerate(out):
                top = torch.topk(logits[i], 2).values
                if float(top[0] - top[1]) > floor:
                    assert token == int(logits[i].argmax()), (len(prompt), i)
                    checked += 1
        print(which, "tokens checked against the plain model:", checked, "of", new * len(prompts))
        assert checked >= 3
        # a stop token in the middle of request 0
        eos = base[0][7]
        stopped = {}
        for graphs, ahead in ((False, False), (True, True)):
            engine = Engine.from_pretrained(folder, cuda_graphs=graphs, lookahead=ahead, eos_token_id=eos, **options)
            stopped[graphs] = engine.generate(prompts, SamplingParams(max_new_tokens=new))
            assert engine.request("req-0").finish_reason == "stop" and engine.cache.free_pages() == [100]
        assert stopped[True] == stopped[False]
        cut = base[0].index(eos) + 1
        assert stopped[True][0] == base[0][:cut]
        for i in (1, 2):
            want = base[i][: base[i].index(eos) + 1] if eos in base[i] else base[i]
            assert stopped[True][i] == want
    finally:
        shutil.rmtree(tmp_path, ignore_errors=True)


def test_cuttings_agree_with_each_other_at_real_layer_sizes_bf16(tmp_path):
    """The same request whole, in portions and with its tail decoded, at the 2.2B layer sizes in
    bfloat16: the three differ from each other by far less than each differs from the 32-bit plain
    model (the tensor-core prefill kernel, the decode kernels and the products of many and of few rows
    all meet here)."""
    import shutil

    folder = folder_for(tmp_path, "2b", "bfloat16")
    try:
        cfg = plain.read_config(folder)
        seq = helpers.random_sequence(cfg["vocab"], 300, 21)
        places = list(range(0, 300, 13)) + [268, 269, 299]
        trace = helpers.Trace()
        trace.sequences.update({"w": seq, "p": seq, "t": seq})
        trace.add_step([("w", 300, places)], end=["w"])
        fed = 0
        for n in (130, 2, 65, 3, 100):
            trace.add_step([("p", n, [p - fed for p in places if fed <= p < fed + n])], end=["p"] if fed + n == 300 else [])
            fed += n
        trace.add_step([("t", 268, [p for p in places if p < 268])])
        for i in range(268, 300):
            trace.add_step([("t", 1, [0] if i in places else [])], end=["t"] if i == 299 else [])
        results = helpers.run_trace(folder, "bfloat16", trace, tmp_path / "out")
        stats = helpers.cuttings_agree(trace, results, ["w", "p", "t"], places=places)
        print("2b sizes bfloat16, whole against portions and tail:", stats)
        assert stats["max_fraction"] <= helpers.BF16_AGREE_FRACTION, stats
        assert stats["mean_fraction"] <= helpers.BF16_AGREE_MEAN_FRACTION, stats
    finally:
        shutil.rmtree(tmp_path, ignore_errors=True)


def test_products_tuned_before_a_capture_change_no_clear_token(tmp_path):
    """``tune_products``: the second time a layout with 1,024 rows or more is seen, the library's proposals for
    its products are timed before the layout is captured.  The trials run (the library counts them), prompts of
    equal length go through the eager step, the tuned eager step and the replayed graph, and every token
    is the plain model's wherever its top-2 margin is clear."""
    import shutil

    from edgerag_b200 import Engine, SamplingParams
    from edgerag_b200.ops import kernels

    folder = folder_for(tmp_path, "2b", "bfloat16")
    try:
        cfg, weights = plain.read_config(folder), plain.read_weights(folder)
        engine = Engine.from_pretrained(folder, dtype="bfloat16", block_size=16, num_blocks=80, chunk_size=1100, max_batch_size=1,
                                        tune_products=True)
        prompts = [helpers.random_sequence(cfg["vocab"], 1040, 700 + i) for i in range(3)]
        trials_before = kernels.linear_trials(torch.bfloat16)
        outs = [engine.generate([p], SamplingParams(max_new_tokens=3))[0] for p in prompts]     # one after the other: the same layouts
        assert engine.runner.graph_replays >= 1
        assert kernels.linear_trials(torch.bfloat16) >= trials_before + 4, "no trials ran"     # q/k/v, output, gate/up, down
        checked = 0
        for prompt, out in zip(prompts, outs):
            logits = plain.forward(weights, cfg, prompt + out[:-1])[len(prompt) - 1:]
            floor = 0.05 * float(logits.abs().max())
            for i, token in enumerate(out):
                top = torch.topk(logits[i], 2).values
                if float(top[0] - top[1]) > floor:
                    assert token == int(logits[i].argmax()), i
                    checked += 1
        assert checked >= 3
    finally:
        shutil.rmtree(tmp_path, ignore_errors=True)


@pytest.mark.parametrize("which", ["2b", "500m"])
def test_a_request_decodes_to_the_same_bits_whatever_shares_its_step(which, tmp_path):
    """Requests with the same prompt (each prefilled alone, so their caches hold the same bits in different
    pages) decode the same token: one alone, one beside 7 others, one beside 15.  The logits are equal bit
    for bit: up to 16 rows the products of a decode step add a row's terms in an order that does not depend
    on the number of rows, the norms and the rotary epilogue work row by row, and with ``batch_invariant``
    the attention kernel cuts every sequence into the same splits and groups of heads whatever the batch
    (the twins' context spans two splits).  Beside 31 and 63 others the
    layers' products are the library's (whose sums depend on the number of rows) and, for the attention
    output and the down projection, this package's partial sums over slices of k that the next norm adds:
    there the logits agree within the band of two cuttings of a request."""
    import shutil

    from edgerag_b200 import Engine
    from edgerag_b200.engine.step import StepEntry

    folder = folder_for(tmp_path, which, "bfloat16")
    try:
        cfg = plain.read_config(folder)
        engine = Engine.from_pretrained(folder, dtype="bfloat16", block_size=16, num_blocks=70 * 8 + 5 * 40, max_batch_size=70,
                                        max_step_tokens=640, cuda_graphs=False, batch_invariant=True)
        runner = engine.runner
        same = helpers.random_sequence(cfg["vocab"], 600, 5)
        twins = [f"x{i}" for i in range(5)]
        others = [f"o{i}" for i in range(63)]
        for i, rid in enumerate(twins + others):
            runner.admit(rid)
            prompt = same if rid in twins else helpers.random_sequence(cfg["vocab"], 40 + (7 * i) % 70, 100 + i)
            runner.step([StepEntry(rid, tokens=prompt)])
        rows = {}
        for twin, beside in zip(twins, (0, 7, 15, 31, 63)):
            entries = [StepEntry(o, tokens=[11 + n]) for n, o in enumerate(others[:beside])]
            entries.insert(beside // 2, StepEntry(twin, tokens=[321], want=[0]))       # somewhere in the middle of the batch
            rows[beside] = runner.step(entries)[0].clone()
        torch.cuda.synchronize()
        assert torch.isfinite(rows[0]).all()
        from edgerag_b200.ops import kernels
        act = torch.empty((32, cfg["inter"]), dtype=torch.bfloat16, device="cuda")
        assert kernels.linear_parts_count(act, engine.model.blocks[0].ffn.w_down) >= 2      # 32 and 64 rows took that path
        for beside in (7, 15):
            differ = int((rows[beside] != rows[0]).sum())
            assert differ == 0, f"beside {beside} others: {differ} of {rows[0].numel()} logits differ"
        scale = float(rows[0].abs().max())
        for beside in (31, 63):
            diff = (rows[beside] - rows[0]).abs()
            assert float(diff.max()) <= helpers.BF16_AGREE_FRACTION * scale and float(diff.mean()) <= helpers.BF16_AGREE_MEAN_FRACTION * scale
    finally:
        shutil.rmtree(tmp_path, ignore_errors=True)
