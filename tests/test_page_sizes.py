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
