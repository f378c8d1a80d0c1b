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


@pytest.mark.parametrize("which,dtype", [("2b", "bfloat16"), ("2b", "float32"), ("256m", "bfloat16"), ("256m", "float32"),
                                         ("500m", "bfloat16")])
def test_cuttings_at_real_layer_sizes(which, dtype, tmp_path):
    folder = folder_for(tmp_path, which, dtype)
    cfg = plain.read_config(folder)
    trace = helpers.Trace()
    base = {"s0": helpers.random_sequence(cfg["vocab"], 333, 1), "s1": helpers.random_sequence(cfg["vocab"], 140, 2),
            "s2": helpers.random_sequence(cfg["vocab"], 70, 3)}
    for tag in ("whole", "tail", "portions", "mixed"):
        for rid, seq in base.items():
            trace.sequences[f"{tag}-{rid}"] = seq

    def want_last(n):      # logits of a few places per step keep the files small at a 49k vocabulary
        return sorted({0, n - 1, n // 2})

    for rid in base:
        n = trace.remaining(f"whole-{rid}")
        trace.add_step([(f"whole-{rid}", n, want_last(n))], end=[f"whole-{rid}"])
    n = trace.remaining("tail-s0")
    trace.add_step([("tail-s0", n - 32, want_last(n - 32))])
    for i in range(32):
        trace.add_step([("tail-s0", 1, "all")], end=["tail-s0"] if i == 31 else [])
    sizes = (130, 2, 65, 3, 128, 5)
    i = 0
    while trace.remaining("portions-s0"):
        n = min(sizes[i % len(sizes)], trace.remaining("portions-s0"))
        if trace.remaining("portions-s0") - n == 1:
            n += 1
        trace.add_step([("portions-s0", n, want_last(n))], end=["portions-s0"] if trace.remaining("portions-s0") == n else [])
        i += 1
    # mixed: portions of one request beside single tokens of the others, pages reused afterwards
    trace.add_step([("mixed-s0", 200, [199]), ("mixed-s1", 100, [99])])
    trace.add_step([("mixed-s0", 1, "all"), ("mixed-s1", 39, [38]), ("mixed-s2", 50, [49])])
    for _ in range(20):
        trace.add_step([("mixed-s0", 1, "all"), ("mixed-s1", 1, "all") if trace.remaining("mixed-s1") else ("mixed-s2", 1, "all")])
    trace.add_step([("mixed-s0", trace.remaining("mixed-s0"), "last")], end=["mixed-s0", "mixed-s1"])
    trace.add_step([("mixed-s2", trace.remaining("mixed-s2"), "last")], end=["mixed-s2"])

    try:
        results = helpers.run_trace(folder, dtype, trace, tmp_path / "out", extra=("--poison-freed-pages",))
        reference = helpers.plain_reference(folder, {k: v for k, v in trace.sequences.items()
                                                     if any(k == e[2] for e in trace.expect)})
        stats = helpers.compare(trace, results, reference, dtype, label=f"{which} sizes")
        print(which, dtype, stats)
    finally:
        import shutil

        shutil.rmtree(tmp_path, ignore_errors=True)      # up to a gigabyte of weights and logits
