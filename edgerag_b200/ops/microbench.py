"""Time one kernel of the engine in isolation, on the device clock, against its roofline.

    python -m edgerag_b200.ops.microbench decode-attention --batch 8 --context 8192
    python -m edgerag_b200.ops.microbench prefill-attention --tokens 2048
    python -m edgerag_b200.ops.microbench linear --m 8 --n 6144 --k 2048
    python -m edgerag_b200.ops.microbench step-kernels --layers 4 --batch 8 --context 8192 --iters 4

Each case builds random inputs larger than the 126 MB L2 where the real workload is (or says that
it is not), runs warm-up launches, then times ``--iters`` launches replayed from one CUDA graph with
CUDA events and prints one JSON line with the median per launch.  Fractions are of the peaks in a
JSON file ``{"hbm_gbs": ..., "bf16_tflops": ...}`` named by ``--peaks`` or, by default,
``MEASURED_PEAKS.json`` in the working directory or beside the package; without such a file they
are of the stated defaults, and the line says which (``"peaks"``).
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys
from pathlib import Path

import torch

from . import kernels

HBM_GBS, BF16_TFLOPS = 6650.0, 1590.0   # defaults (a B200's copy bandwidth and library bf16 product rate) when no file is found
PEAKS_FROM = "defaults"


def load_peaks(path: str | None) -> None:
    """Take the roofline denominators from a JSON file of measured peaks, if there is one."""
    global HBM_GBS, BF16_TFLOPS, PEAKS_FROM
    candidates = [Path(path)] if path else [Path.cwd() / "MEASURED_PEAKS.json",
                                            Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"]
    for cand in candidates:
        try:
            raw = json.loads(cand.read_text())
            HBM_GBS, BF16_TFLOPS, PEAKS_FROM = float(raw["hbm_gbs"]), float(raw["bf16_tflops"]), f"measured ({cand.name})"
            return
        except (OSError, KeyError, ValueError):
            continue
    if path:
        raise SystemExit(f"--peaks {path}: not a JSON file with hbm_gbs and bf16_tflops")


def _time(fn, iters: int, warmup: int, rounds: int = 5) -> float:
    """Median over ``rounds`` of the time per launch of ``iters`` launches, in microseconds.  The launches
    are captured into one CUDA graph and replayed, so that kernels of a few microseconds are timed
    back to back as they run inside a step, not at the rate the host can issue them."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(iters):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(rounds):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3 / iters)
    return statistics.median(times)


def _paged(batch: int, context: int, nkv: int, d: int, page: int, dtype, shuffle: bool = True):
    """Key and value pools of ``batch`` sequences of ``context`` tokens with their block tables."""
    pages_per = -(-context // page)
    n_pages = batch * pages_per
    kp = torch.randn((n_pages, nkv, page, d), device="cuda", dtype=torch.float32).to(dtype)
    vp = torch.randn((n_pages, nkv, page, d), device="cuda", dtype=torch.float32).to(dtype)
    order = torch.randperm(n_pages) if shuffle else torch.arange(n_pages)
    tables = order.view(batch, pages_per).to(torch.int32).cuda()
    return kp, vp, tables


def decode_attention(a) -> dict:
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    nbytes = 2 * a.batch * a.context * a.kv_heads * a.head_dim * (2 if dtype == torch.bfloat16 else 4)
    # --cold: rotate over so many caches that each launch finds its keys and values in DRAM, as a
    # step does whose weights have passed through L2 since the layer's cache was last read
    reps = max(2, int(300e6 // nbytes) + 1) if a.cold else 1
    caches = [_paged(a.batch, a.context, a.kv_heads, a.head_dim, a.page, dtype, not a.sequential_pages) for _ in range(reps)]
    state = {"i": 0}

    def cache():
        state["i"] = (state["i"] + 1) % reps
        return caches[state["i"]]

    q = torch.randn((a.batch, a.heads * a.head_dim), device="cuda").to(dtype)
    out = torch.empty_like(q)
    pos = torch.full((a.batch,), a.context - 1, dtype=torch.int32, device="cuda")
    tok = torch.arange(a.batch, dtype=torch.int32, device="cuda")
    if a.split <= 0:        # as the engine chooses it: from the batch and a power-of-two bound on the context
        bound, granule = kernels.context_bound(-(-a.context // a.page))
        a.split, heads = kernels.choose_decode_plan(a.batch, a.kv_heads, bound * a.page, a.page, a.head_dim, a.kernel != "bulk",
                                                    granule * a.page)
        a.head_group = a.head_group or heads
    splits = (a.context - 1) // a.split + 1
    acc_n, ml_n = kernels.decode_scratch_floats(a.batch, a.heads, a.head_dim, splits)
    acc, ml = torch.empty(acc_n, device="cuda"), torch.empty(ml_n, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    scale = a.head_dim ** -0.5
    if a.kernel == "gqa":
        fn = lambda: kernels.attention_decode_gqa(q, *cache(), tok, pos, out, a.heads, scale, acc, ml, splits,  # noqa: E731
                                                  status, split_keys=a.split)
    elif a.kernel == "bulk":
        fn = lambda: kernels.attention_decode_bulk(q, *cache(), tok, pos, out, a.heads, scale, acc, ml, splits,  # noqa: E731
                                                   status, split_keys=a.split, head_group=a.head_group)
    else:
        fn = lambda: kernels.attention_decode(q, *cache(), tok, pos, out, a.heads, scale, acc, ml, splits,  # noqa: E731
                                              split_keys=a.split)
    us = _time(fn, max(a.iters, 2 * reps), a.warmup)
    return {"case": "decode-attention", "kernel": a.kernel, "split": a.split, "head_group": a.head_group, "us": round(us, 2),
            "bytes": nbytes, "gbs": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / HBM_GBS, 4),
            "status": int(status), "from_dram": bool(a.cold) or nbytes > 126e6}


def prefill_attention(a) -> dict:
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    total = a.past + a.tokens
    kp, vp, tables = _paged(1, total, a.kv_heads, a.head_dim, a.page, dtype, not a.sequential_pages)
    width = (a.heads + 2 * a.kv_heads) * a.head_dim
    qkv = torch.randn((a.tokens, width), device="cuda").to(dtype)
    out = torch.empty((a.tokens, a.heads * a.head_dim), device="cuda", dtype=dtype)
    pos = torch.arange(a.past, total, dtype=torch.int32, device="cuda")
    starts = torch.tensor([0, a.tokens], dtype=torch.int32, device="cuda")
    seq_of = torch.zeros(a.tokens, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    scale = a.head_dim ** -0.5
    if a.kernel == "tc":
        blocks = kernels.prefill_tc_blocks([a.tokens])
        ranges = a.key_splits or kernels.prefill_tc_key_splits(blocks, a.heads, total, qkv.device)
        need_o, need_ml = kernels.prefill_tc_scratch_floats(a.tokens, a.heads, ranges)
        part_o, part_ml = torch.empty(need_o, device="cuda"), torch.empty(need_ml, device="cuda")
        fn = lambda: kernels.attention_prefill_tc(qkv, kp, vp, tables, starts, pos, out, blocks, a.heads, scale, status,  # noqa: E731
                                                  key_splits=ranges, part_o=part_o, part_ml=part_ml)
    else:
        fn = lambda: kernels.attention_rows(qkv, kp, vp, tables, seq_of, pos, out, a.heads, scale)  # noqa: E731
    us = _time(fn, a.iters, a.warmup)
    pairs = a.tokens * a.past + a.tokens * (a.tokens + 1) / 2
    flops = 4.0 * a.heads * a.head_dim * pairs
    return {"case": "prefill-attention", "kernel": a.kernel, "us": round(us, 2), "tflops": round(flops / us / 1e6, 1),
            "frac_bf16": round(flops / us / 1e6 / BF16_TFLOPS, 4), "status": int(status)}


def linear(a) -> dict:
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    reps = max(1, int(200e6 // (a.n * a.k * 2)) + 1)    # rotate over several weight copies: more than L2 in total
    ws = [torch.randn((a.n, a.k), device="cuda").to(dtype) for _ in range(reps)]
    x = torch.randn((a.m, a.k), device="cuda").to(dtype)
    out = torch.empty((a.m, a.n), device="cuda", dtype=torch.float32 if a.out32 else dtype)
    out_glu = torch.empty((a.m, a.n // 2), device="cuda", dtype=dtype) if a.glu else None
    n_parts = kernels.linear_parts_slices(ws[0]) if a.parts else 0
    parts = torch.empty((n_parts, a.m, a.n), device="cuda", dtype=torch.float32) if n_parts else None
    state = {"i": 0}

    def fn():
        state["i"] = (state["i"] + 1) % reps
        if a.parts:
            kernels.linear_parts(x, ws[state["i"]], parts)
        elif a.tc:
            (kernels.linear_tc_glu if a.glu else kernels.linear_tc)(x, ws[state["i"]], out_glu if a.glu else out)
        elif a.glu:
            kernels.linear_glu(x, ws[state["i"]], out_glu)
        else:
            kernels.linear(x, ws[state["i"]], out, library=a.library)

    us = _time(fn, a.iters, a.warmup)
    nbytes = a.n * a.k * x.element_size() + a.m * a.k * x.element_size() + out.numel() * out.element_size()
    flops = 2.0 * a.m * a.n * a.k
    if n_parts:
        nbytes += parts.numel() * 4 - out.numel() * out.element_size()
    return {"case": "linear", "m": a.m, "n": a.n, "k": a.k, "library": bool(a.library), "tc": bool(a.tc), "glu": bool(a.glu), "parts": n_parts, "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1),
            "frac_hbm": round(nbytes / us / 1e3 / HBM_GBS, 4), "tflops": round(flops / us / 1e6, 2)}


def step_kernels(a) -> dict:
    """Which kernels a step's time goes to: the SmolVLM-2.2B layer sizes with ``--layers`` layers, a
    prefill of ``--tokens`` tokens and decode steps of ``--batch`` sequences at ``--context``, run
    eagerly under the CUDA activity tracer without chained launches (so that a kernel's time is its
    own).  The microseconds are per launch and carry the tracer's overhead: read them as shares."""
    import os

    os.environ["EDGERAG_B200_NO_CHAIN"] = "1"          # read when the first library launches a kernel
    from torch.profiler import ProfilerActivity, profile

    from ..engine.engine import Engine, EngineOptions
    from ..engine.step import StepEntry

    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": a.layers, "hidden_size": 2048,
           "num_attention_heads": a.heads, "num_key_value_heads": a.kv_heads, "head_dim": 64, "intermediate_size": 8192,
           "vocab_size": 49155, "rope_theta": 273768.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
           "hidden_act": "silu", "max_position_embeddings": 8192, "pad_token_id": 0}
    eng = Engine.from_config(cfg, 0, 0.02, EngineOptions(
        dtype="bfloat16", block_size=16, num_blocks=a.batch * (a.context // 16 + 2) + a.tokens // 16 + 64,
        max_batch_size=a.batch + 2, chunk_size=a.tokens, max_step_tokens=a.tokens + a.batch, max_model_len=a.context + 8,
        cuda_graphs=False))
    r = eng.runner
    ids = torch.randint(0, 49155, (a.tokens,)).tolist()

    def table(prof, launches_of):
        rows = [(e.key, e.device_time_total / max(1, e.count), e.count) for e in prof.key_averages() if e.device_time_total > 0]
        total = sum(us * n for _, us, n in rows)
        rows.sort(key=lambda x: -x[1] * x[2])
        return {"total_us_per_" + launches_of[0]: round(total / launches_of[1], 1),
                "kernels": [{"name": k[:70], "us": round(us, 2), "calls": n, "share": round(us * n / total, 3)} for k, us, n in rows[:12]]}

    def prefill(name):
        r.admit(name)
        r.step([StepEntry(name, tokens=ids, want=[a.tokens - 1])])
        r.release(name)

    prefill("w0")
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as p1:
        prefill("w1")
        torch.cuda.synchronize()
    names = [f"d{i}" for i in range(a.batch)]
    for n in names:
        r.admit(n)
        eng.cache.grow(n, a.context - 64)
        eng.cache.advance(n, a.context - 64)
    for _ in range(3):
        r.step([StepEntry(n, tokens=[5], want=[0]) for n in names])
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as p2:
        for _ in range(a.iters):
            r.step([StepEntry(n, tokens=[5], want=[0]) for n in names])
        torch.cuda.synchronize()
    return {"case": "step-kernels", "layers": a.layers, "batch": a.batch, "context": a.context, "tokens": a.tokens,
            "prefill": table(p1, ("step", 1)), "decode": table(p2, ("step", a.iters))}


def step_timeline(a) -> dict:
    """Where a decode step's time goes when its kernels run as they do in serving: replayed from a CUDA
    graph with chained launches, so that a kernel starts while the one before it drains.  The activity
    tracer gives every kernel's start and end; a kernel's share of the critical path is the time from
    the end of the kernels before it to its own end.  ``--layers`` layers of the SmolVLM-2.2B sizes,
    ``--batch`` sequences at ``--context``; averages over the layers after the first, in microseconds
    (they carry the tracer's overhead: read them as shares)."""
    from torch.profiler import ProfilerActivity, profile

    from ..engine.engine import Engine, EngineOptions
    from ..engine.step import StepEntry

    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": a.layers, "hidden_size": 2048,
           "num_attention_heads": a.heads, "num_key_value_heads": a.kv_heads, "head_dim": 64, "intermediate_size": 8192,
           "vocab_size": 49155, "rope_theta": 273768.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
           "hidden_act": "silu", "max_position_embeddings": 8192, "pad_token_id": 0}
    eng = Engine.from_config(cfg, 0, 0.02, EngineOptions(
        dtype="bfloat16", block_size=16, num_blocks=a.batch * (a.context // 16 + 2) + 64, max_batch_size=a.batch + 2,
        max_step_tokens=512 + a.batch, max_model_len=a.context + 8, cuda_graphs=True))
    r = eng.runner
    names = [f"d{i}" for i in range(a.batch)]
    for n in names:
        r.admit(n)
        eng.cache.grow(n, a.context - 16)
        eng.cache.advance(n, a.context - 16)
    step = lambda: r.step([StepEntry(n, tokens=[5], want=[0]) for n in names])  # noqa: E731
    for _ in range(4):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step()
        torch.cuda.synchronize()
    events = sorted((e for e in prof.events() if "cuda" in str(e.device_type).lower() and "Memcpy" not in e.name),
                    key=lambda e: e.time_range.start)
    first = max(i for i, e in enumerate(events) if "embed_rows" in e.name)
    events = events[first:]
    names_of = [e.name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0][:48] for e in events]
    norms = [i for i, n in enumerate(names_of) if n.startswith("add_rmsnorm")]
    per_layer = norms[2] - norms[0] if len(norms) > 2 else len(events) - 1      # a layer: from its first norm to the next layer's
    t0, frontier = events[0].time_range.start, events[0].time_range.end
    shares: dict[tuple[int, str], list[float]] = {}
    starts = []
    for i, e in enumerate(events[1: 1 + per_layer * a.layers]):
        if i % per_layer == 0:
            starts.append(e.time_range.start)
        name = names_of[1 + i]
        shares.setdefault((i % per_layer, name), []).append(max(0.0, e.time_range.end - max(frontier, e.time_range.start)))
        frontier = max(frontier, e.time_range.end)
    rows = [{"kernel": name, "critical_us": round(sum(v[1:]) / max(1, len(v) - 1), 2)} for (_, name), v in sorted(shares.items())]
    period = (starts[-1] - starts[0]) / max(1, len(starts) - 1) if len(starts) > 1 else 0.0
    return {"case": "step-timeline", "layers": a.layers, "batch": a.batch, "context": a.context, "replayed_from_graph": r.graph_replays > 0,
            "layer_period_us": round(period, 2), "step_us": round(events[-1].time_range.end - t0, 1), "kernels_of_a_layer": rows}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="edgerag_b200.ops.microbench", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="case", required=True)
    common = argparse.ArgumentParser(add_help=False)
    common.add_argument("--iters", type=int, default=20)
    common.add_argument("--warmup", type=int, default=3)
    common.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    common.add_argument("--peaks", default=None, help="JSON file with hbm_gbs and bf16_tflops to take fractions of")
    att = argparse.ArgumentParser(add_help=False)
    att.add_argument("--heads", type=int, default=32)
    att.add_argument("--kv-heads", type=int, default=32)
    att.add_argument("--head-dim", type=int, default=64)
    att.add_argument("--page", type=int, default=16)
    att.add_argument("--sequential-pages", action="store_true", help="pages in order instead of shuffled")
    d = sub.add_parser("decode-attention", parents=[common, att])
    d.add_argument("--batch", type=int, default=8)
    d.add_argument("--context", type=int, default=8192)
    d.add_argument("--split", type=int, default=0, help="keys per split; 0: the engine's choice for this batch")
    d.add_argument("--kernel", choices=["bulk", "gqa", "general"], default="bulk")
    d.add_argument("--head-group", type=int, default=0, help="kv heads per block of the bulk kernel; 0: its own choice")
    d.add_argument("--cold", action="store_true", help="rotate over several caches so that none is found in L2")
    p = sub.add_parser("prefill-attention", parents=[common, att])
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--past", type=int, default=0)
    p.add_argument("--key-splits", type=int, default=0, help="ranges every block's keys are cut into; 0: the engine's choice")
    p.add_argument("--kernel", choices=["tc", "general"], default="tc")
    g = sub.add_parser("linear", parents=[common])
    g.add_argument("--m", type=int, default=8)
    g.add_argument("--n", type=int, default=6144)
    g.add_argument("--k", type=int, default=2048)
    g.add_argument("--out32", action="store_true")
    g.add_argument("--library", action="store_true", help="force the library product (cuBLASLt) also for few rows")
    g.add_argument("--tc", action="store_true", help="the TMA + tcgen05 weight-streaming kernel (up to 64 rows)")
    g.add_argument("--parts", action="store_true", help="the slices of k as float32 partial results (17 to 64 rows, a weight of few rows)")
    g.add_argument("--glu", action="store_true", help="the gated product: w is [gate; up] of n rows, out has n / 2 columns")
    k = sub.add_parser("step-kernels", parents=[common])
    k.add_argument("--layers", type=int, default=4)
    k.add_argument("--batch", type=int, default=8)
    k.add_argument("--context", type=int, default=8192)
    k.add_argument("--tokens", type=int, default=2048)
    k.add_argument("--heads", type=int, default=32)
    k.add_argument("--kv-heads", type=int, default=32)
    t = sub.add_parser("step-timeline", parents=[common])
    t.add_argument("--layers", type=int, default=4)
    t.add_argument("--batch", type=int, default=8)
    t.add_argument("--context", type=int, default=640)
    t.add_argument("--heads", type=int, default=32)
    t.add_argument("--kv-heads", type=int, default=32)
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("microbench needs a CUDA device", file=sys.stderr)
        return 1
    fn = {"decode-attention": decode_attention, "prefill-attention": prefill_attention, "linear": linear,
          "step-kernels": step_kernels, "step-timeline": step_timeline}[a.case]
    load_peaks(a.peaks)
    result = fn(a)
    result["peaks"] = PEAKS_FROM
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
