"""The plain implementation against the golden outputs of the reference's own decoder."""

from __future__ import annotations

from pathlib import Path

import pytest
import torch
from safetensors.torch import load_file

import plain_llama as plain

GOLDEN = Path(__file__).resolve().parent / "golden"
CASES = {"a": (plain.TINY_A, 0, 0.05, 16), "b": (plain.TINY_B, 1, 0.08, 8)}


@pytest.mark.parametrize("tag", ["a", "b"])
def test_plain_matches_reference_decoder(tag, tmp_path):
    raw, seed, std, n_new = CASES[tag]
    folder = plain.write_model_folder(tmp_path / tag, raw, seed, std=std)
    cfg, weights = plain.read_config(folder), plain.read_weights(folder)
    golden = load_file(str(GOLDEN / f"golden_tiny_{tag}.safetensors"))
    n_prompts = sum(1 for k in golden if k.startswith("prompt_"))
    assert n_prompts >= 2
    for i in range(n_prompts):
        prompt = golden[f"prompt_{i}"].tolist()
        logits = plain.forward(weights, cfg, prompt)
        want = golden[f"logits_{i}"]
        torch.testing.assert_close(logits[-want.shape[0]:], want, atol=1e-6, rtol=1e-6)
        greedy = plain.greedy_generate(weights, cfg, prompt, n_new)
        assert greedy == golden[f"greedy_{i}"].tolist()[:n_new]
        # what the reference's scheduler and executor generate for the same prompts served together, in
        # prompt portions of 4, 8 and 64 tokens (edgerag tests/test_executor.py:120-191)
        for chunk in (4, 8, 64):
            assert golden[f"served_chunk{chunk}_{i}"].tolist() == greedy


def test_embeds_path_equals_ids_path(tmp_path):
    """edgerag tests/test_executor.py:247-265: feeding the embedding rows equals feeding the ids."""
    folder = plain.write_model_folder(tmp_path / "b", plain.TINY_B, 1, std=0.08)
    cfg, weights = plain.read_config(folder), plain.read_weights(folder)
    ids = torch.randint(0, cfg["vocab"], (19,), generator=torch.Generator().manual_seed(3))
    a = plain.forward(weights, cfg, ids.tolist())
    b = plain.forward(weights, cfg, embeds=plain.embed(weights, ids))
    torch.testing.assert_close(a, b, atol=0, rtol=0)
    with pytest.raises(ValueError):
        plain.forward(weights, cfg)


def test_parts_landmines():
    """repeat_kv repeats consecutively, the mask uses finfo.min, rotate_half is the halves convention
    (edgerag tests/test_equivalence.py:330-383)."""
    x = torch.arange(3.0).view(3, 1, 1)
    assert plain.repeat_kv(x, 2).flatten().tolist() == [0, 0, 1, 1, 2, 2]
    m = plain.causal_mask(3, torch.float32, "cpu")
    assert m[0, 1] == torch.finfo(torch.float32).min and m[1, 0] == 0 and m[2, 2] == 0
    assert plain.rotate_half(torch.tensor([1.0, 2.0, 3.0, 4.0])).tolist() == [-3, -4, 1, 2]
    w = plain.causal_mask(5, torch.float32, "cpu", window=2)
    assert (w[4] == 0).tolist() == [False, False, False, True, True]


def test_temperature_reference():
    logits = torch.tensor([0.0, 1.0, 2.0])
    p = plain.temperature_probs(logits, 0.5)
    assert abs(float(p.sum()) - 1) < 1e-12 and p[2] > p[1] > p[0]
    assert plain.inverse_cdf_pick(p, 0.0) == 0
    assert plain.inverse_cdf_pick(p, float(p[0]) + 1e-9) == 1
    assert plain.inverse_cdf_pick(p, 0.999999) == 2
