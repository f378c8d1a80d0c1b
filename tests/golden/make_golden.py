"""Make the golden outputs of tests/golden/: logits of Tejas544/edgerag's own decoder on tiny models.

Run once, on the CPU, with the reference checkout importable:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference /path/to/edgerag

For each tiny configuration of ``tests/plain_llama.py`` it writes a model folder with seeded
random weights (in a temporary directory), loads the same tensors into the reference's
``EdgeRagDecoder(spec, use_eager=True)`` (edgerag/core/model.py:31-152, built in fp32 from
``FP16Linear``, which despite its name is a plain ``nn.Linear`` wrapper, edgerag/core/linear.py:70-104),
runs whole prompts through it, and stores a subset of the logits rows, the greedy continuation
produced with the reference's own paged cache (edgerag/cache/paged.py), the prompts, and the greedy
tokens of all prompts served together by the reference's own scheduler and executor with prompt
portions of 4, 8 and 64 tokens (``served_chunk<c>_<i>``).  It also
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
CHUNKS = (4, 8, 64)  # prompt portions of the reference's executor (tests/test_executor.py:120-160)


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


@torch.inference_mode()
def reference_scheduled(spec, model, prompts: list[list[int]], n_new: int, block_size: int, chunk: int) -> list[list[int]]:
    """Greedy tokens of all prompts served together by the reference's own ``Scheduler`` and
    ``ModelExecutor`` (edgerag/sched/scheduler.py:95-309, edgerag/serve/executor.py:57-165) with prompt
    portions of ``chunk`` tokens, driven by the threadless loop of its tests
    (tests/test_executor.py:54-70): schedule, execute, report portions and tokens, end the step."""
    from edgerag.cache.allocator import BlockAllocator
    from edgerag.sched.request import Request
    from edgerag.sched.scheduler import Scheduler, SchedulerConfig
    from edgerag.serve.executor import ModelExecutor

    allocator = BlockAllocator(256, block_size)
    executor = ModelExecutor(model, spec, allocator, torch.device("cpu"), torch.float32, chunk_size=chunk)
    scheduler = Scheduler(allocator, SchedulerConfig(max_batch_size=len(prompts), prefill_chunk_size=chunk,
                                                     cow_reserve_blocks=0, max_prefills_per_step=1))
    requests = [Request(request_id=f"g{i}", prompt_token_ids=list(p), max_new_tokens=n_new) for i, p in enumerate(prompts)]
    for r in requests:
        scheduler.add_request(r)
    for _ in range(10000):
        if not scheduler.has_work:
            break
        batch = scheduler.schedule()
        out = executor.execute(batch)
        for r in batch.requests:
            n = out.prefilled.get(r.request_id, 0)
            if n:
                scheduler.on_prefill_chunk(r, n)
            t = out.tokens.get(r.request_id)
            if t is not None:
                scheduler.on_token(r, t)
        scheduler.end_step()
    assert all(len(r.generated_token_ids) == n_new for r in requests), [len(r.generated_token_ids) for r in requests]
    return [list(r.generated_token_ids) for r in requests]


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
        prompts = prompts_for(case, cfg["vocab"])
        for chunk in CHUNKS:
            served = reference_scheduled(spec, model, prompts, case["n_new"], 8 if tag == "b" else 16, chunk)
            for i, tokens in enumerate(served):
                out[f"served_chunk{chunk}_{i}"] = torch.tensor(tokens, dtype=torch.int32)
        save_file(out, str(HERE / f"golden_tiny_{tag}.safetensors"))
        print(f"tiny {tag}: max |reference - plain| = {worst:.3e}; logits scale {float(ref.abs().max()):.3f}")


if __name__ == "__main__":
    main()
