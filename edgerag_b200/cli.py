"""Command line: generate from a model folder, or from seeded random weights.

    python -m edgerag_b200 --model DIR --prompt-ids 1,2,3 --max-new-tokens 16
    python -m edgerag_b200 --random-weights 0 --config config.json --save-model DIR --prompt-ids 1,2,3

Options the reference's launcher has keep their names and meanings (scripts/serve_rag.py:104-131):
``--model`` (here a folder, there a hub id), ``--budget-gib`` (size the page pool from a memory
budget; 0: use ``--num-blocks``), ``--num-blocks``, ``--chunk-size``, ``--device``; the engine knobs
of its ``SchedulerConfig`` (edgerag/sched/scheduler.py:40-49) are ``--max-batch-size``,
``--max-prefills-per-step`` and ``--eos-token-id``.  Its quantisation, retrieval and HTTP options
(``--arm --bits --group-size -k --host --port``) have no counterpart: those parts are not built.
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path


def _parse_ids(text: str) -> list[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="edgerag_b200", description="Generate tokens with the B200 engine")
    src = ap.add_argument_group("model")
    src.add_argument("--model", help="folder with config.json and model.safetensors")
    src.add_argument("--random-weights", type=int, metavar="SEED", help="use seeded random weights (needs --config)")
    src.add_argument("--config", help="config.json for --random-weights")
    src.add_argument("--save-model", metavar="DIR", help="with --random-weights: write the model folder here first")
    src.add_argument("--weights-std", type=float, default=0.02)
    ap.add_argument("--dtype", choices=["bf16", "fp32", "bfloat16", "float32"], default="bf16")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--budget-gib", type=float, default=0.0,
                    help="size the page pool so that the engine stays within this much device memory; 0: --num-blocks")
    ap.add_argument("--num-blocks", type=int, default=None, help="pages in the pool (default: --kv-fraction of free memory)")
    ap.add_argument("--kv-fraction", type=float, default=0.8)
    ap.add_argument("--chunk-size", type=int, default=512, help="prompt tokens per request per step")
    ap.add_argument("--max-batch-size", type=int, default=8)
    ap.add_argument("--max-prefills-per-step", type=int, default=1)
    ap.add_argument("--max-model-len", type=int, default=None)
    ap.add_argument("--max-new-tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--eos-token-id", type=int, default=None)
    ap.add_argument("--no-lookahead", action="store_true",
                    help="read every step's tokens before the next step is launched")
    ap.add_argument("--no-cuda-graphs", action="store_true", help="launch every kernel of every step from the host")
    ap.add_argument("--batch-invariant", action="store_true",
                    help="kernel shapes that do not follow the batch: the same bits for a request whatever shares its step")
    ap.add_argument("--tune-products", action="store_true",
                    help="time the library's algorithms for large products once before a step layout is captured (for long runs of equal large steps)")
    ap.add_argument("--prompt-ids", action="append", default=[], metavar="IDS",
                    help="a prompt as token ids, comma or space separated; may be given several times")
    ap.add_argument("--prompt-file", help="a file with one prompt per line (token ids)")
    ap.add_argument("--json", action="store_true", help="print one JSON line instead of text")
    return ap


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    if (args.model is None) == (args.random_weights is None):
        print("give exactly one of --model and --random-weights", file=sys.stderr)
        return 2
    prompts = [_parse_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        prompts += [_parse_ids(l) for l in Path(args.prompt_file).read_text().splitlines() if l.strip()]
    if not prompts:
        print("no prompt: use --prompt-ids or --prompt-file", file=sys.stderr)
        return 2

    from .engine.engine import Engine, EngineOptions
    from .sampling.params import SamplingParams

    options = EngineOptions(
        dtype=args.dtype, device=args.device, block_size=args.block_size, num_blocks=args.num_blocks,
        budget_gib=args.budget_gib or None, kv_fraction=args.kv_fraction, max_batch_size=args.max_batch_size,
        chunk_size=args.chunk_size, max_prefills_per_step=args.max_prefills_per_step,
        max_model_len=args.max_model_len, eos_token_id=args.eos_token_id, seed=args.seed,
        lookahead=not args.no_lookahead, cuda_graphs=not args.no_cuda_graphs, batch_invariant=args.batch_invariant,
        tune_products=args.tune_products)
    t0 = time.perf_counter()
    if args.model is not None:
        engine = Engine.from_pretrained(args.model, options)
    else:
        if not args.config:
            print("--random-weights needs --config", file=sys.stderr)
            return 2
        raw = json.loads(Path(args.config).read_text())
        if args.save_model:
            import torch

            from .config.registry import architecture_of
            from .engine.engine import resolve_dtype
            from .models.decoder import DecoderModel
            from .weights.loader import write_model_folder

            arch = architecture_of(raw)
            plan = arch.make_plan(arch.read_config(raw, args.config))
            specs = DecoderModel(plan, torch.float32, torch.device("cpu")).weight_specs()
            write_model_folder(args.save_model, raw, specs, args.random_weights, std=args.weights_std,
                               dtype=resolve_dtype(args.dtype))
            engine = Engine.from_pretrained(args.save_model, options)
        else:
            engine = Engine.from_config(raw, args.random_weights, args.weights_std, options)
    t_load = time.perf_counter() - t0
    params = SamplingParams(temperature=args.temperature, seed=args.seed if args.temperature > 0 else None,
                            max_new_tokens=args.max_new_tokens)
    t0 = time.perf_counter()
    outputs = engine.generate(prompts, params)
    t_gen = time.perf_counter() - t0
    n_new = sum(len(o) for o in outputs)
    if args.json:
        print(json.dumps({
            "outputs": [{"prompt_len": len(p), "token_ids": o} for p, o in zip(prompts, outputs)],
            "load_s": round(t_load, 3), "generate_s": round(t_gen, 3), "new_tokens": n_new,
            "scheduler": engine.scheduler.stats.to_dict()}))
    else:
        for i, (p, o) in enumerate(zip(prompts, outputs)):
            print(f"[{i}] prompt of {len(p)} tokens -> {' '.join(map(str, o))}")
        print(f"{n_new} tokens in {t_gen:.3f} s ({n_new / max(t_gen, 1e-9):.1f} tok/s); load {t_load:.2f} s", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
