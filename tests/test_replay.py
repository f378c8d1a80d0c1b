"""Replay through bin/trace_run under every cutting, in 32-bit and in bfloat16, against the plain model.

The same requests are fed whole; with the last 32 tokens one by one; in portions of changing
size down to two tokens; and mixed, up to four live requests with portions of some beside single
tokens of others, in a pool that is exactly as large as the trace needs so that pages are used
again.  One process per (model, dtype) replays all of them in a row, so that later scenarios run
in pages that earlier ones left behind.
"""

from __future__ import annotations

import numpy as np
import pytest

import helpers
import plain_llama as plain

pytestmark = pytest.mark.gpu

LENGTHS = {"a": (7, 33, 150, 97), "b": (5, 40, 77, 131)}
BLOCK = {"a": 16, "b": 8}


def build_trace(which: str, vocab: int) -> helpers.Trace:
    trace = helpers.Trace()
    base = {f"s{i}": helpers.random_sequence(vocab, n, 100 + i) for i, n in enumerate(LENGTHS[which])}
    for tag in ("whole", "tail", "portions", "mixed"):
        for rid, seq in base.items():
            trace.sequences[f"{tag}-{rid}"] = seq
    for rid in base:
        helpers.cut_whole(trace, f"whole-{rid}")
    for rid, seq in base.items():
        if len(seq) > 40:
            helpers.cut_tail_decode(trace, f"tail-{rid}", tail=32)
    for rid in base:
        helpers.cut_portions(trace, f"portions-{rid}")
    # two rounds of mixing so that more than four requests pass through the pool
    trace.sequences.update({f"mixed2-{rid}": seq[::-1] for rid, seq in base.items()})
    helpers.cut_mixed(trace, [f"mixed-{rid}" for rid in base] + [f"mixed2-{rid}" for rid in base], seed=7)
    return trace


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b"])
def test_all_cuttings_match_plain(which, dtype, model_folders, tmp_path):
    folder = model_folders(which, dtype)
    cfg = plain.read_config(folder)
    trace = build_trace(which, cfg["vocab"])
    results = helpers.run_trace(folder, dtype, trace, tmp_path / "out", block_size=BLOCK[which],
                                extra=("--poison-freed-pages",))
    reference = helpers.plain_reference(folder, trace.sequences)
    stats = helpers.compare(trace, results, reference, dtype, label=f"tiny {which}")
    print(f"tiny {which} {dtype}: {len(trace.steps)} steps, {len(trace.expect)} rows, {stats}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decode(dtype, model_folders, tmp_path):
    """Logits at positions 0, 1, 2 of a sequence, then 300 tokens decoded one by one across many pages."""
    folder = model_folders("a", dtype)
    cfg = plain.read_config(folder)
    trace = helpers.Trace()
    trace.sequences["long"] = helpers.random_sequence(cfg["vocab"], 303, 5)
    trace.add_step([("long", 1, "all")])
    trace.add_step([("long", 2, "all")])
    for _ in range(300):
        trace.add_step([("long", 1, "all")])
    results = helpers.run_trace(folder, dtype, trace, tmp_path / "out", extra=("--poison-freed-pages",))
    helpers.compare(trace, results, helpers.plain_reference(folder, trace.sequences), dtype, "long decode")


def test_cuttings_agree_with_each_other_bf16(model_folders, tmp_path):
    """In bfloat16 the cuttings differ from each other by the rounding of a few sums only (the order in
    which a product or a softmax adds its terms), far less than any of them differs from the 32-bit
    plain model, where every activation's rounding counts.  The band is a few times the difference
    that was measured, an order of magnitude below the band of the comparison with the plain model."""
    folder = model_folders("b", "bfloat16")
    cfg = plain.read_config(folder)
    seq = helpers.random_sequence(cfg["vocab"], 90, 11)
    trace = helpers.Trace()
    trace.sequences.update({"w": seq, "p": seq, "t": seq})
    helpers.cut_whole(trace, "w")
    helpers.cut_portions(trace, "p")
    helpers.cut_tail_decode(trace, "t", tail=32)
    results = helpers.run_trace(folder, "bfloat16", trace, tmp_path / "out", block_size=8)
    stats = helpers.cuttings_agree(trace, results, ["w", "p", "t"], len(seq))
    print("tiny b bfloat16, whole against portions and tail:", stats)
    assert stats["max_fraction"] <= helpers.BF16_AGREE_FRACTION, stats
    assert stats["mean_fraction"] <= helpers.BF16_AGREE_MEAN_FRACTION, stats
