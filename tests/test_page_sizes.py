"""Greedy generation through the entry point with cache pages of 8 to 128 tokens: the kernels that a page
size selects (whole pages per bulk copy, pages per TMA tile, pages that do or do not divide a stage)
all have to give the plain model's tokens."""

from __future__ import annotations

import pytest
import torch

import plain_llama as plain

WIDE = dict(plain.TINY_A, hidden_size=256, num_attention_heads=4, num_key_value_heads=4, head_dim=64,
            intermediate_size=512, vocab_size=1000, max_position_embeddings=2048)
GROUPED = dict(WIDE, num_attention_heads=6, num_key_value_heads=2, hidden_size=384)


@pytest.mark.gpu
@pytest.mark.parametrize("name,config,std", [("heads of 64", WIDE, 0.08), ("grouped heads of 64", GROUPED, 0.08),
                                             ("tiny A", plain.TINY_A, 0.2), ("tiny B", plain.TINY_B, 0.2)])
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_generation_with_every_page_size(name, config, std, dtype, tmp_path):
    import shutil

    from edgerag_b200 import Engine, SamplingParams

    folder = plain.write_model_folder(tmp_path, config, seed=0, std=std, dtype=getattr(torch, dtype))
    try:
        cfg, weights = plain.read_config(folder), plain.read_weights(folder)
        longest = 700 if cfg["head_dim"] == 64 else 200
        prompts = [[(7 * i + 3) % cfg["vocab"] for i in range(longest)], [(11 * i + 5) % cfg["vocab"] for i in range(70)],
                   [(13 * i + 1) % cfg["vocab"] for i in range(min(300, longest))]]
        margin = 0.05 if dtype == "bfloat16" else 1e-3
        judged = []
        for prompt in prompts:      # where the plain model's choice is clear, given the tokens before
            judged.append(lambda out, p=prompt: plain.forward(weights, cfg, list(p) + out[:-1])[len(p) - 1:])
        for page in (8, 16, 32, 64, 128):
            for graphs in (False, True):
                engine = Engine.from_pretrained(folder, dtype=dtype, block_size=page, num_blocks=max(24, 3 * 1200 // page), chunk_size=256,
                                                max_batch_size=4, max_prefills_per_step=2, cuda_graphs=graphs, poison_freed_pages=True)
                outs = engine.generate(prompts, SamplingParams(max_new_tokens=12))
                checked = 0
                for rows_of, out in zip(judged, outs):
                    for got, row in zip(out, rows_of(out)):
                        top = torch.topk(row, 2).values
                        if float(top[0] - top[1]) >= margin * float(row.abs().max()):
                            assert got == int(row.argmax()), f"{name}, pages of {page}, graphs {graphs}"
                            checked += 1
                assert checked >= 12, "too few clear choices to judge by"
    finally:
        shutil.rmtree(tmp_path, ignore_errors=True)


ODD = [
    dict(hidden_size=100, num_attention_heads=5, num_key_value_heads=5, head_dim=16, intermediate_size=100, vocab_size=257),
    dict(hidden_size=72, num_attention_heads=3, num_key_value_heads=1, head_dim=48, intermediate_size=250, vocab_size=1001),
    dict(hidden_size=136, num_attention_heads=7, num_key_value_heads=7, head_dim=80, intermediate_size=136, vocab_size=300),
    dict(hidden_size=200, num_attention_heads=6, num_key_value_heads=3, head_dim=112, intermediate_size=264, vocab_size=515),
    dict(hidden_size=256, num_attention_heads=2, num_key_value_heads=2, head_dim=128, intermediate_size=512, vocab_size=999),
    dict(hidden_size=192, num_attention_heads=9, num_key_value_heads=3, head_dim=64, intermediate_size=320, vocab_size=777),
    dict(hidden_size=64, num_attention_heads=1, num_key_value_heads=1, head_dim=256, intermediate_size=96, vocab_size=130),
    dict(hidden_size=90, num_attention_heads=10, num_key_value_heads=2, head_dim=32, intermediate_size=70, vocab_size=64),
]


@pytest.mark.gpu
@pytest.mark.parametrize("sizes", ODD, ids=lambda c: f"h{c['hidden_size']}-{c['num_attention_heads']}x{c['head_dim']}")
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_generation_with_sizes_that_are_no_powers_of_two(sizes, dtype, tmp_path):
    """Widths, head counts, head sizes in steps of 16 up to 256, intermediate sizes and vocabularies that are
    no powers of two (some no multiple of 8, where the vector kernels give way to the scalar ones and the
    weight-streaming products to the library): every combination gives the plain model's tokens."""
    import shutil

    from edgerag_b200 import Engine, SamplingParams

    config = dict(plain.TINY_A, **sizes, max_position_embeddings=1024)
    folder = plain.write_model_folder(tmp_path, config, seed=sizes["hidden_size"], std=0.12, dtype=getattr(torch, dtype))
    try:
        cfg, weights = plain.read_config(folder), plain.read_weights(folder)
        v = cfg["vocab"]
        prompts = [[(7 * k + 3) % v for k in range(300)], [(11 * k + 5) % v for k in range(40)], [(13 * k + 1) % v for k in range(17)]]
        margin = 0.05 if dtype == "bfloat16" else 1e-3
        for graphs in (False, True):
            engine = Engine.from_pretrained(folder, dtype=dtype, block_size=16, num_blocks=64, chunk_size=128, max_batch_size=4,
                                            max_prefills_per_step=2, cuda_graphs=graphs, poison_freed_pages=True)
            outs = engine.generate(prompts, SamplingParams(max_new_tokens=10))
            checked = 0
            for prompt, out in zip(prompts, outs):
                logits = plain.forward(weights, cfg, list(prompt) + out[:-1])[len(prompt) - 1:]
                for got, row in zip(out, logits):
                    top = torch.topk(row, 2).values
                    if float(top[0] - top[1]) >= margin * float(row.abs().max()):
                        assert got == int(row.argmax()), f"{sizes}, graphs {graphs}"
                        checked += 1
            assert checked >= 10, "too few clear choices to judge by"
    finally:
        shutil.rmtree(tmp_path, ignore_errors=True)
