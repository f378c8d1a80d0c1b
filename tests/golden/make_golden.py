"""Make the golden outputs of tests/golden/: logits of Tejas544/edgerag's own decoder on tiny models.

Run once, on the CPU, with the reference checkout importable:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference /path/to/edgerag

For each tiny configuration of ``tests/plain_llama.py`` it writes a model folder with seeded
random weights (in a temporary directory), loads the same tensors into the reference's
``EdgeRagDecoder(spec, use_eager=True)`` (edgerag/core/model.py:31-152, built in fp32 from
``FP16Linear``, which despite its name is a plain ``nn.Linear`` wrapper, edgerag/core/linear.py:70-104),
runs whole prompts through it, and stores a subset of the logits rows, the greedy continuation
produced with the reference's own paged cache (edgerag/cache/paged.py), and the prompts.  It also
prints the largest difference between the reference and ``plain_llama.forward`` on those prompts.

The committed ``golden_tiny_*.safetensors`` files were made by this script; ``tests/test_plain.py``
checks the plain implementation against them, so the oracle of the suite is anchored on the
reference's code and not only on a reading of its formulas.
"""

from __future__ import annotations

import argparse
import sys
import tempfile
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import plain_llama as plain  # noqa: E402

CASES = {
    "a": dict(raw=plain.TINY_A, seed=0, std=0.05, prompt_lens=(7, 33), n_new=16),
    "b": dict(raw=plain.TINY_B, seed=1, std=0.08, prompt_lens=(5, 40, 77), n_new=8),
}
ROWS = 12  # logits rows kept per prompt (the last ones)


def prompts_for(case: dict, vocab: int) -> list[list[int]]:
    gen = torch.Generator().manual_seed(1000 + case["seed"])
    return [torch.randint(0, vocab, (n,), generator=gen).tolist() for n in case["prompt_lens"]]


def build_reference(cfg: dict, weights: dict):
    from edgerag.core.model import EdgeRagDecoder
    from edgerag.core.spec import ModelSpec

    spec = ModelSpec(
        model_id="tiny", model_type="smolvlm", n_layers=cfg["n_layers"], hidden_size=cfg["hidden"],
        n_q_heads=cfg["n_q"], n_kv_heads=cfg["n_kv"], head_dim=cfg["head_dim"], vocab_size=cfg["vocab"],
        max_position_embeddings=512, rope_theta=cfg["theta"], vision_layers=1, vision_hidden=8,
        vision_image_size=16, vision_patch_size=8, scale_factor=1, image_token_id=1, pad_token_id=0,
        rms_norm_eps=cfg["eps"], intermediate_size=cfg["inter"], hidden_act="silu",
    )
    model = EdgeRagDecoder(spec, use_eager=True).eval().to(torch.float32)
    state = {}
    for name, tensor in weights.items():
        key = name.removeprefix("model.")
        if key.endswith("_proj.weight") or key == "lm_head.weight":
            key = key[: -len("weight")] + "linear.weight"
        state[key] = tensor
    if "lm_head.linear.weight" not in state:
        state["lm_head.linear.weight"] = state["embed_tokens.weight"]
    missing, unexpected = model.load_state_dict(state, strict=False)
    assert not unexpected and all("inv_freq" in m for m in missing), (missing, unexpected)
    return spec, model


@torch.inference_mode()
def reference_greedy(spec, model, prompt: list[int], n_new: int, block_size: int) -> list[int]:
    from edgerag.cache.allocator import BlockAllocator
    from edgerag.cache.paged import PagedKVCache

    cache = PagedKVCache(spec, BlockAllocator(64, block_size), torch.device("cpu"), torch.float32)
    logits = model(input_ids=torch.tensor([prompt]), cache=cache, last_token_only=True)
    out = []
    for _ in range(n_new):
        token = int(logits[0, -1].argmax())
        out.append(token)
        logits = model(input_ids=torch.tensor([[token]]), cache=cache, last_token_only=True)
    return out


def main() -> None:
    from safetensors.torch import save_file

    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of Tejas544/edgerag")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)

    for tag, case in CASES.items():
        with tempfile.TemporaryDirectory() as tmp:
            folder = plain.write_model_folder(tmp, case["raw"], case["seed"], std=case["std"])
            cfg = plain.read_config(folder)
            weights = plain.read_weights(folder)
        spec, model = build_reference(cfg, weights)
        out, worst = {}, 0.0
        for i, prompt in enumerate(prompts_for(case, cfg["vocab"])):
            with torch.inference_mode():
                ref = model(input_ids=torch.tensor([prompt]))[0]
            mine = plain.forward(weights, cfg, prompt)
            worst = max(worst, float((ref - mine).abs().max()))
            out[f"prompt_{i}"] = torch.tensor(prompt, dtype=torch.int32)
            out[f"logits_{i}"] = ref[-ROWS:].contiguous()
            out[f"greedy_{i}"] = torch.tensor(
                reference_greedy(spec, model, prompt, case["n_new"], block_size=8 if tag == "b" else 16),
                dtype=torch.int32,
            )
        save_file(out, str(HERE / f"golden_tiny_{tag}.safetensors"))
        print(f"tiny {tag}: max |reference - plain| = {worst:.3e}; logits scale {float(ref.abs().max()):.3f}")


if __name__ == "__main__":
    main()
