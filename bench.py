#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of the SmolVLM-2.2B decoder (24 layers, hidden 2048, 32 query
and 32 key/value heads of 64, intermediate 8192, vocabulary 49155, rope theta 273768, eps 1e-5,
tied head), random bfloat16 weights, cache pages of 16 tokens, a batch of 8 requests and a context
of 8192 tokens.  A "step" is one decode step of the whole batch.

* ``value``: decoded tokens per second, timed on the device with CUDA events around K steps of the
  step function plus the sampling kernel, fed from the host with fixed token ids.
* ``e2e``: the same through the Python entry point (``Engine.step``): host token ids in, sampled
  token ids out, every step, timed by the wall clock between two synchronisations.
* ``prefill``: one step with a portion of 2,048 prompt tokens.
* ``roofline``: bytes the decode step has to read (every weight once, the cache of the live
  requests) over its time, against the measured copy bandwidth.
* ``points``: decode throughput at batch 1 and 64 with the same context, and at batch 1, 8 and 64
  with a short context of 640 tokens (``decode_b8_ctx640`` ...), where the weights dominate the bytes.
* ``spread`` (and ``*_p50_ms`` / ``*_std_ms`` beside every point): every timed step is a trial of its
  own (an event after each), reported as median, 95th percentile and standard deviation; the prefill
  is the median of five runs.

The step's inputs (3.4 GB of weights, 12.9 GB of cache at batch 8) are far larger than the 126 MB
L2, so no flush is needed between timed iterations.  ``--impl reference`` runs the unmodified
reference package installed under ``baseline/_ref`` through its own scheduler and executor.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent

CONFIG_2B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 24, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 32, "head_dim": 64, "intermediate_size": 8192,
    "vocab_size": 49155, "rope_theta": 273768.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 8192, "hidden_act": "silu", "pad_token_id": 0,
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            out = {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"])}
            if raw.get("bf16_tflops_sustained"):
                out["bf16_tflops_sustained"] = float(raw["bf16_tflops_sustained"])
            return out, "measured"
        except (KeyError, ValueError, json.JSONDecodeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Reads SM clocks and throttle reasons through NVML while a timed region runs (reads only)."""

    REASONS = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
               0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
               0x100: "display_clock_setting"}

    def __init__(self, index: int = 0, period: float = 0.05) -> None:
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._period = period
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:  # no NVML: the record says so
            self._nv = None

    def _loop(self) -> None:
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self._period)

    def __enter__(self) -> "ClockSampler":
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def merge(self, other: "ClockSampler") -> None:
        self.samples += other.samples
        self.reasons |= other.reasons

    def record(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml_unavailable"]}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons)}


def spread(samples_ms: list[float]) -> dict:
    """Median, 95th percentile and standard deviation of per-trial times (the reference reports p50,
    p95 and std over at least five trials and refuses a single number: bench/bench.py:159-227,
    bench/metrics.py:165-200)."""
    xs = sorted(samples_ms)
    p95 = xs[min(len(xs) - 1, int(math.ceil(0.95 * len(xs))) - 1)]
    return {"trials": len(xs), "p50_ms": round(statistics.median(xs), 4), "p95_ms": round(p95, 4),
            "std_ms": round(statistics.pstdev(xs), 4) if len(xs) > 1 else 0.0}


def model_numbers(cfg: dict, n_layers: int) -> dict:
    h, d = cfg["hidden_size"], cfg["head_dim"]
    nq, nkv, inter, vocab = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"], cfg["vocab_size"]
    per_layer = h * d * (nq + 2 * nkv) + nq * d * h + 3 * h * inter
    return {
        "linear_params": n_layers * per_layer,
        "head_params": vocab * h,
        "norm_params": (2 * n_layers + 1) * h,
        "kv_bytes_per_token": 2 * n_layers * nkv * d * 2,
        "attn_flops_per_pair": 4 * nq * d * n_layers,     # q.k and p.v, per (query, visible key)
    }


def decode_bytes(nums: dict, context_lens: list[int]) -> float:
    """Bytes one decode step must read: every weight once (bf16; norm weights float32) and the live cache."""
    weights = 2 * (nums["linear_params"] + nums["head_params"]) + 4 * nums["norm_params"]
    return weights + nums["kv_bytes_per_token"] * float(sum(context_lens))


def run_ours(args) -> dict:
    import torch

    sys.path.insert(0, str(ROOT))
    from edgerag_b200.engine.engine import Engine, EngineOptions
    from edgerag_b200.engine.step import StepEntry
    from edgerag_b200.ops import kernels
    from edgerag_b200.sampling.params import SamplingParams

    torch.cuda.set_device(0)
    cfg = dict(CONFIG_2B)
    cfg["num_hidden_layers"] = args.layers
    context, batch, block = args.context, args.batch, 16
    nums = model_numbers(cfg, args.layers)
    peak, peak_source = peaks()
    point_batches = [] if args.no_points else [1, 64]
    most = max([batch] + point_batches)
    pages_per_seq = context // block + 2
    engine = Engine.from_config(cfg, weights_seed=0, std=0.02, options=EngineOptions(
        dtype="bfloat16", device="cuda:0", block_size=block, num_blocks=most * pages_per_seq + 8 + 2048 // block,
        max_batch_size=most + 1, chunk_size=2048, max_prefills_per_step=batch, max_step_tokens=2048 * batch + most,
        max_model_len=context + 8, tune_products=True))     # (the prefill step's layout is captured: its products are tuned once)
    runner, cache = engine.runner, engine.cache
    vocab = cfg["vocab_size"]
    gen = torch.Generator().manual_seed(0)
    clocks = ClockSampler()

    def timed_decode(entries_fn, steps: int, warmup: int) -> tuple[float, int, dict]:
        """K decode steps of the step function plus sampling, on the device clock.  An event after every
        step makes each step a trial of its own.  Returns (ms/step over the whole region, own launches,
        spread of the K per-step times)."""
        tokens = torch.empty(256, dtype=torch.int32, device="cuda")
        for _ in range(warmup):
            kernels.sample_rows(runner.step(entries_fn()), tokens)
        torch.cuda.synchronize()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        before = kernels.launch_counts["own"]
        sampler = ClockSampler()
        with sampler:
            marks[0].record()
            for i in range(steps):
                kernels.sample_rows(runner.step(entries_fn()), tokens)
                marks[i + 1].record()
            torch.cuda.synchronize()
        clocks.merge(sampler)
        per_step = [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]
        return marks[0].elapsed_time(marks[steps]) / steps, kernels.launch_counts["own"] - before, spread(per_step)

    # --- prefill: one step with 2,048 prompt tokens -------------------------------------------------
    prefill_tokens = 2048
    ids = torch.randint(0, vocab, (prefill_tokens,), generator=gen).tolist()
    times = []
    for i in range(9):
        runner.admit(f"p{i}")
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        runner.step([StepEntry(f"p{i}", tokens=ids, want=[prefill_tokens - 1])])
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        runner.release(f"p{i}")
    # five trials after four warm-up runs (in the fourth the library's proposals for the shapes are timed, as in serving)
    prefill_spread = spread(times[4:])
    prefill_ms = prefill_spread["p50_ms"]
    pairs = prefill_tokens * (prefill_tokens + 1) / 2
    prefill_flops = 2.0 * prefill_tokens * nums["linear_params"] + 2.0 * nums["head_params"] + nums["attn_flops_per_pair"] * pairs
    prefill = {"value": round(prefill_tokens / (prefill_ms / 1e3), 1), "tokens": prefill_tokens, "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4),
               "tflop": round(prefill_flops / 1e12, 3), "ms_min": round(min(times[4:]), 3),
               "std_ms": prefill_spread["std_ms"], "trials": prefill_spread["trials"]}

    # --- the headline: batch 8 at the full context, through the entry point --------------------------
    k, w = args.steps, args.warmup
    prompt_len = context - (2 * (k + w) + 4)
    for i in range(batch):
        engine.add_request(torch.randint(0, vocab, (prompt_len,), generator=gen).tolist(),
                           SamplingParams(max_new_tokens=2 * (k + w) + 4), request_id=f"d{i}")
    while any(engine.request(f"d{i}").pending > 1 or engine.request(f"d{i}").num_computed == 0 for i in range(batch)):
        engine.step()
    for _ in range(w):
        engine.step()
    torch.cuda.synchronize()
    sampler = ClockSampler()
    h2d = d2h = 0
    e2e_steps = []
    with sampler:
        t0 = last = time.perf_counter()
        for _ in range(k):
            events = engine.step()
            h2d += runner.h2d_bytes_last
            d2h += engine.d2h_bytes_last
            now = time.perf_counter()
            e2e_steps.append(1e3 * (now - last))
            last = now
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
    clocks.merge(sampler)
    if len(events) != batch:
        raise RuntimeError(f"{len(events)} of {batch} requests were decoding in the timed steps")
    e2e = {"value": round(batch * k / e2e_s, 1), "unit": "tokens/s", "ms_per_step": round(1e3 * e2e_s / k, 4),
           "h2d_bytes_per_step": h2d // k, "d2h_bytes_per_step": d2h // k,
           **{f"step_{key}": v for key, v in spread(e2e_steps).items() if key != "trials"}}

    # the same requests, driven below the scheduler with fixed ids, on the device clock
    live = [f"d{i}" for i in range(batch)]
    fixed = torch.randint(0, vocab, (batch,), generator=gen).tolist()
    ms_per_step, launches, step_spread = timed_decode(
        lambda: [StepEntry(r, tokens=[t], want=[0]) for r, t in zip(live, fixed)], k, w)
    ctx_lens = [cache.requests[r].num_tokens for r in live]
    need = decode_bytes(nums, ctx_lens)
    achieved = need / (ms_per_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peak["hbm_gbs"], 4), "bytes_per_step": int(need)}
    value = batch / (ms_per_step / 1e3)
    for r in live:
        engine.scheduler.abort(engine.request(r), "bench_done")

    # --- points: batch 1 and 64 at the same context (cache filled without running the prompts) --------
    # Then the same batches and batch 8 at a short context (prompts of 512 tokens plus some generated ones),
    # where the step is bound by the weights, not the cache.
    points = {}
    short = 640
    for pb, ctx in [(b, context) for b in point_batches] + ([(b, short) for b in (1, batch, 64)] if point_batches else []):
        names = [f"b{pb}_{ctx}_{i}" for i in range(pb)]
        for r in names:
            runner.admit(r)
            cache.grow(r, ctx - 2 * (k + w) - 4)
            cache.advance(r, ctx - 2 * (k + w) - 4)
        # pages keep what earlier requests wrote: finite bfloat16 values either way
        toks = torch.randint(0, vocab, (pb,), generator=gen).tolist()
        ms, _, sp = timed_decode(lambda: [StepEntry(r, tokens=[t], want=[0]) for r, t in zip(names, toks)], k, w)
        tag = f"decode_b{pb}" if ctx == context else f"decode_b{pb}_ctx{ctx}"
        points[tag] = round(pb / (ms / 1e3), 1)
        points[f"{tag}_ms"] = round(ms, 4)
        points[f"{tag}_p50_ms"], points[f"{tag}_std_ms"] = sp["p50_ms"], sp["std_ms"]
        lens = [cache.requests[r].num_tokens for r in names]
        points[f"{tag}_hbm_frac"] = round(decode_bytes(nums, lens) / (ms / 1e3) / 1e9 / peak["hbm_gbs"], 4)
        for r in names:
            runner.release(r)

    return {
        "metric": "decode_tokens_per_s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": k,
        "warmup": w, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": "SmolVLM-2.2B decoder (random weights)", "global_batch": batch, "seq_len": context,
            "parallelism": "single", "layers": args.layers, "layers_full": CONFIG_2B["num_hidden_layers"],
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": vocab,
            "rope_theta": cfg["rope_theta"], "rms_eps": cfg["rms_norm_eps"], "tied": True, "page_tokens": block,
            "l2": "inputs larger than L2 (weights 3.4 GB + cache), no flush", "points_context": context,
            "peaks": peak_source,
            "cuda_graphs": ("on, tune_products" if engine.options.tune_products else "on") if engine.options.cuda_graphs and runner.graphs_enabled else "off",
        },
        "clocks": clocks.record(), "e2e": e2e, "gpu_launches": int(launches), "prefill": prefill,
        "roofline": roofline, "points": points, "spread": step_spread,
    }


CONFIG_256M = dict(CONFIG_2B, num_hidden_layers=30, hidden_size=576, num_attention_heads=9, num_key_value_heads=3,
                   intermediate_size=1536, vocab_size=49280, rope_theta=100000.0)
CONFIG_500M = dict(CONFIG_2B, num_hidden_layers=32, hidden_size=960, num_attention_heads=15, num_key_value_heads=5,
                   intermediate_size=2560, vocab_size=49280, rope_theta=100000.0)


def run_serving_workload(args) -> dict:
    """The two serving workloads of the smaller SmolVLM decoders, through ``Engine.generate``:

    * ``mixed``: 256M sizes, 32 requests with prompts of 64..4096 tokens, half of them given as
      ``prompt_embeds``, 512-token portions beside decode tokens, 64 new tokens each;
    * ``continuous``: 500M sizes, 64 requests of 7,472 prompt tokens and 128 new tokens, the page
      pool sized to 80 % of the free memory.
    """
    import torch

    sys.path.insert(0, str(ROOT))
    from edgerag_b200.engine.engine import Engine, EngineOptions
    from edgerag_b200.sampling.params import SamplingParams

    torch.cuda.set_device(0)
    gen = torch.Generator().manual_seed(0)
    if args.workload == "mixed":
        cfg, n_req, new = CONFIG_256M, 32, 64
        lens = torch.randint(64, 4097, (n_req,), generator=gen).tolist()
        options = EngineOptions(dtype="bfloat16", block_size=16, kv_fraction=0.5, max_batch_size=32, chunk_size=512,
                                max_prefills_per_step=2)
    else:
        cfg, n_req, new = CONFIG_500M, 64, 128
        lens = [7472] * n_req
        options = EngineOptions(dtype="bfloat16", block_size=16, kv_fraction=0.8, max_batch_size=64, chunk_size=512,
                                max_prefills_per_step=2)
    engine = Engine.from_config(cfg, weights_seed=0, std=0.02, options=options)
    prompts, embeds = [], []
    for i, n in enumerate(lens):
        prompts.append(torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist())
        use_rows = args.workload == "mixed" and i % 2 == 1
        embeds.append(torch.randn((n, cfg["hidden_size"]), generator=gen).to(torch.bfloat16).cuda() if use_rows else None)
    warm = engine.generate([prompts[0][:600]], SamplingParams(max_new_tokens=4))   # compiles, sizes buffers
    assert len(warm[0]) == 4
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    with ClockSampler() as clocks:
        outs = engine.generate(prompts, SamplingParams(max_new_tokens=new), prompt_embeds=embeds)
        torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    generated = sum(len(o) for o in outs)
    stats = engine.scheduler.stats.to_dict()
    return {
        "metric": f"{args.workload}_serving_tokens_per_s", "value": round((sum(lens) + generated) / wall, 1),
        "unit": "tokens/s (prompt + generated)", "generated_tokens_per_s": round(generated / wall, 1), "wall_s": round(wall, 3),
        "n_gpus": 1, "dtype": "bf16", "data": "synthetic", "impl": "ours", "higher_is_better": True,
        "config": {"model": "SmolVLM-256M decoder" if args.workload == "mixed" else "SmolVLM-500M decoder",
                   "requests": n_req, "prompt_tokens": sum(lens), "new_tokens_each": new, "chunk": 512,
                   "pool_pages": engine.cache.pages[0].capacity, "page_tokens": 16,
                   "embeds_requests": sum(e is not None for e in embeds)},
        "scheduler": stats, "clocks": clocks.record(),
        "graphs": {"captured": len(engine.runner._graphs), "replays": engine.runner.graph_replays},
    }


def run_reference(args) -> dict:
    """The unmodified reference: its decoder, paged cache, scheduler and executor, random weights, float16."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "edgerag").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip install --no-deps --target baseline/_ref)"}
    sys.path.insert(0, str(ref))
    try:
        import torch
        from edgerag.cache.allocator import BlockAllocator
        from edgerag.core.model import EdgeRagDecoder
        from edgerag.core.spec import ModelSpec
        from edgerag.sched.request import Request, RequestState
        from edgerag.sched.scheduler import Scheduler, SchedulerConfig
        from edgerag.serve.executor import ModelExecutor
    except Exception as exc:  # the package does not import here
        return {"impl": "reference", "unavailable": f"reference import failed: {type(exc).__name__}: {exc}"[:200]}
    on_cpu = bool(getattr(args, "ref_cpu_check", False))    # a small dry run of this function on the CPU
    if not on_cpu and not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device"}

    c = dict(CONFIG_2B)
    if on_cpu:
        c.update(hidden_size=64, num_attention_heads=4, num_key_value_heads=4, head_dim=16, intermediate_size=128,
                 vocab_size=300)
    context, batch, block = args.context, args.batch, 16
    k, w = args.steps, args.warmup
    device = torch.device("cpu" if on_cpu else "cuda:0")
    ref_dtype = torch.float32 if on_cpu else torch.float16
    spec = ModelSpec(
        model_id="bench-2.2b", model_type="smolvlm", n_layers=args.layers, hidden_size=c["hidden_size"],
        n_q_heads=c["num_attention_heads"], n_kv_heads=c["num_key_value_heads"], head_dim=c["head_dim"],
        vocab_size=c["vocab_size"], max_position_embeddings=context, rope_theta=c["rope_theta"], vision_layers=1,
        vision_hidden=8, vision_image_size=16, vision_patch_size=8, scale_factor=1, image_token_id=1, pad_token_id=0,
        rms_norm_eps=c["rms_norm_eps"], intermediate_size=c["intermediate_size"], hidden_act="silu")
    torch.manual_seed(0)
    with torch.device(device):
        decoder = EdgeRagDecoder(spec).eval().to(ref_dtype)
    for p in decoder.parameters():
        if p.dim() > 1:
            p.data.normal_(0.0, 0.02)
    allocator = BlockAllocator(batch * (context // block + 2) + 8, block)
    executor = ModelExecutor(decoder, spec, allocator, device, ref_dtype, chunk_size=512)
    scheduler = Scheduler(allocator, SchedulerConfig(max_batch_size=batch, prefill_chunk_size=512,
                                                     cow_reserve_blocks=4, max_prefills_per_step=1))
    gen = torch.Generator().manual_seed(0)
    # The reference admits one prompt per step and decodes the earlier requests meanwhile, so request i
    # has generated about chunks * (batch - 1 - i) tokens when the last prompt is in.  Prompts are
    # shortened by that much, so that every request is near the full context in the timed steps and
    # none runs out of new tokens before them.
    chunks = -(-context // 512)
    requests = []
    for i in range(batch):
        ahead = chunks * (batch - 1 - i)
        new_tokens = ahead + k + w + 4
        prompt_len = context - new_tokens
        requests.append(Request(request_id=f"d{i}", max_new_tokens=new_tokens + 64,
                                prompt_token_ids=torch.randint(0, c["vocab_size"], (prompt_len,), generator=gen).tolist()))
    for r in requests:
        scheduler.add_request(r)

    def one_step() -> int:
        b = scheduler.schedule()
        out = executor.execute(b)
        made = 0
        for r in b.requests:
            n = out.prefilled.get(r.request_id, 0)
            if n:
                scheduler.on_prefill_chunk(r, n)
            t = out.tokens.get(r.request_id)
            if t is not None:
                scheduler.on_token(r, t)
                made += 1
        scheduler.end_step()
        return made

    for _ in range(chunks * batch + 64):
        if all(r.state is RequestState.DECODING for r in requests):
            break
        one_step()
    else:
        return {"impl": "reference", "unavailable": "the reference's requests did not all reach decoding"}
    for _ in range(w):
        one_step()
    sync = (lambda: None) if on_cpu else torch.cuda.synchronize
    sync()
    clocks = ClockSampler()
    if not on_cpu:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with clocks:
        t0 = time.perf_counter()
        if not on_cpu:
            start.record()
        made = 0
        for _ in range(k):
            made += one_step()
        if not on_cpu:
            stop.record()
        sync()
        wall = time.perf_counter() - t0
    ms = 1e3 * wall / k if on_cpu else start.elapsed_time(stop) / k
    nums = model_numbers(c, args.layers)
    peak, peak_source = peaks()
    if made != batch * k:
        return {"impl": "reference", "unavailable": f"only {made} of {batch * k} tokens were decoded in the timed steps"}
    need = decode_bytes(nums, [r.total_tokens for r in requests])
    achieved = need / (ms / 1e3) / 1e9
    return {
        "metric": "decode_tokens_per_s", "value": round(made / (ms * k / 1e3), 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": k, "warmup": w, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp16", "data": "synthetic", "impl": "reference",
        "config": {"model": "SmolVLM-2.2B decoder (random weights)", "global_batch": batch, "seq_len": context,
                   "parallelism": "single", "layers": args.layers, "layers_full": c["num_hidden_layers"],
                   "page_tokens": block, "path": "edgerag Scheduler + ModelExecutor (one request at a time)",
                   "peaks": peak_source},
        "clocks": clocks.record(),
        "e2e": {"value": round(made / wall, 1), "unit": "tokens/s", "h2d_bytes_per_step": 8 * batch, "d2h_bytes_per_step": 8 * batch},
        "gpu_launches": 0,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4)},
    }


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONFIG_2B["max_position_embeddings"])
    ap.add_argument("--layers", type=int, default=CONFIG_2B["num_hidden_layers"],
                    help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--workload", choices=["decode", "mixed", "continuous"], default="decode",
                    help="decode: the headline measurement; mixed / continuous: the serving workloads of the "
                         "256M and 500M decoders through Engine.generate")
    ap.add_argument("--ref-cpu-check", action="store_true",
                    help="with --impl reference: a dry run of the reference arm's loop at toy sizes on the CPU")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported (nothing here uses more than one GPU)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        result = run_reference(args)
    elif args.workload != "decode":
        result = run_serving_workload(args)
    else:
        result = run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
