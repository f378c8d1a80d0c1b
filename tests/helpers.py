"""Helpers of the GPU tests: building traces, replaying them through bin/trace_run, comparing."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

import plain_llama as plain

ROOT = Path(__file__).resolve().parent.parent

# Tolerances.  float32: the engine and the plain implementation differ in reduction order only
# (the reference measured 2e-5 between its cached and uncached paths and gates at 1e-4,
# tests/test_equivalence.py:47-57); logits here are O(1).  bfloat16: activations are rounded to 8
# bits of mantissa between the products, so the error is a fraction of the logits' scale.
F32_ATOL, F32_RTOL = 2e-4, 2e-4
BF16_FRACTION = 0.03       # max |error| <= 3 % of the largest |logit| of the row set
BF16_MEAN_FRACTION = 0.005  # mean |error| <= 0.5 % of it


# Two cuttings of the same request in bfloat16 go through the same roundings of activations and differ
# only where a kernel adds its terms in another order (prompt portions against single tokens, a product
# of many rows against one of few): a last-bit difference in one activation, carried through the layers
# above it.  Measured: at most 0.95 % of the largest |logit| and 0.043 % on average at the 2.2B layer
# sizes (0.67 % and 0.008 % on tiny B), where the comparison with the 32-bit plain model shows 2.3 % and
# 0.32 %.  The bands are two to three times what was measured; the mean is the one that tells a fault
# from rounding (a wrong key or a stale page moves every logit of a row).
BF16_AGREE_FRACTION = 0.02
BF16_AGREE_MEAN_FRACTION = 0.0015


def round64(n: int) -> int:
    return -(-n // 64) * 64


class Trace:
    """Steps for bin/trace_run plus the bookkeeping to check their results."""

    def __init__(self) -> None:
        self.steps: list[dict] = []
        self.expect: list[tuple[int, int, str, int]] = []   # (step, row in the step's file, request, position)
        self.sequences: dict[str, list[int]] = {}
        self._fed: dict[str, int] = {}
        self._live: dict[str, int] = {}
        self.max_tokens = 0

    def add_step(self, entries: list[tuple[str, int, list[int] | str]], end: list[str] = ()) -> None:
        """``entries``: (request, n tokens to feed next, wanted places or "all"/"last")."""
        step_no = len(self.steps)
        out, row = [], 0
        for rid, n, want in entries:
            start = self._fed.get(rid, 0)
            toks = self.sequences[rid][start: start + n]
            assert len(toks) == n and n > 0, (rid, start, n)
            places = list(range(n)) if want == "all" else ([n - 1] if want == "last" else list(want))
            out.append({"id": rid, "tokens": toks, "want": places})
            for w in places:
                self.expect.append((step_no, row, rid, start + w))
                row += 1
            self._fed[rid] = start + n
            self._live[rid] = start + n
        self.max_tokens = max(self.max_tokens, sum(round64(c) for c in self._live.values()))
        for rid in end:
            self._live.pop(rid, None)
        self.steps.append({"step": step_no, "entries": out, "end": list(end)})

    def fed(self, rid: str) -> int:
        return self._fed.get(rid, 0)

    def remaining(self, rid: str) -> int:
        return len(self.sequences[rid]) - self.fed(rid)


def run_trace(model_dir: Path, dtype: str, trace: Trace, out_dir: Path, max_tokens: int | None = None,
              block_size: int = 16, extra: tuple[str, ...] = (), timeout: int = 900,
              info: dict | None = None) -> dict[int, np.ndarray]:
    """Pipe the trace through bin/trace_run; return {step: float32 array [wanted, vocab]}.
    ``info``, when given, receives the program's standard error under "stderr"."""
    out_dir.mkdir(parents=True, exist_ok=True)
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens or trace.max_tokens),
           "--block-size", str(block_size), *extra]
    text = "".join(json.dumps(s) + "\n" for s in trace.steps)
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout)
    assert proc.returncode == 0, f"trace_run failed ({proc.returncode}):\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}"
    if info is not None:
        info["stderr"] = proc.stderr
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in trace.steps], "missing 'done' lines"
    vocab = plain.read_config(model_dir)["vocab"]
    results = {}
    for s in trace.steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        f = out_dir / f"{s['step']}.f32"
        if n_want:
            results[s["step"]] = np.fromfile(f, dtype="<f4").reshape(n_want, vocab)
        else:
            assert not f.exists()
    return results


def plain_reference(model_dir: Path, sequences: dict[str, list[int]]) -> dict[str, torch.Tensor]:
    """float32 logits of the plain implementation for every sequence, from the folder's stored values."""
    cfg = plain.read_config(model_dir)
    weights = plain.read_weights(model_dir, torch.float32)
    done: dict[tuple, torch.Tensor] = {}     # requests that feed the same tokens share one computation
    out = {}
    for rid, seq in sequences.items():
        key = tuple(seq)
        if key not in done:
            done[key] = plain.forward(weights, cfg, seq)
        out[rid] = done[key]
    return out


def compare(trace: Trace, results: dict[int, np.ndarray], reference: dict[str, torch.Tensor], dtype: str,
            label: str = "") -> dict[str, float]:
    """Check every wanted row against the plain logits; report the first offender by place."""
    got = np.stack([results[s][row] for s, row, _, _ in trace.expect])
    want = np.stack([reference[rid][pos].numpy() for _, _, rid, pos in trace.expect])
    assert np.isfinite(got).all(), f"{label}: non-finite logits at " + str(
        [trace.expect[i] for i in np.argwhere(~np.isfinite(got).all(axis=1))[:3, 0]])
    err = np.abs(got - want)
    scale = float(np.abs(want).max())
    if dtype == "float32":
        bad = err > F32_ATOL + F32_RTOL * np.abs(want)
    else:
        bad = err > BF16_FRACTION * scale
    if bad.any():
        first = int(np.argwhere(bad.any(axis=1))[0, 0])
        step, row, rid, pos = trace.expect[first]
        raise AssertionError(
            f"{label} [{dtype}]: first wrong place: request {rid} position {pos} (step {step}, row {row}); "
            f"max error there {err[first].max():.3e}, overall {err.max():.3e}, scale {scale:.3f}; "
            f"{int(bad.any(axis=1).sum())} of {len(trace.expect)} rows off")
    if dtype != "float32":
        assert err.mean() <= BF16_MEAN_FRACTION * scale, f"{label}: mean error {err.mean():.3e} vs scale {scale:.3f}"
    return {"max_err": float(err.max()), "mean_err": float(err.mean()), "scale": scale}


def cuttings_agree(trace: Trace, results: dict[int, np.ndarray], rids: list[str], n: int | None = None,
                   places: list[int] | None = None) -> dict[str, float]:
    """Largest and mean difference, as fractions of the largest |logit|, between the logits that the
    requests ``rids`` (the same tokens, cut differently) got at the same positions."""
    rows = {(rid, pos): results[step][row] for step, row, rid, pos in trace.expect if rid in rids}
    places = list(range(n)) if places is None else places
    first = np.stack([rows[(rids[0], i)] for i in places])
    scale = float(np.abs(first).max())
    worst, mean = 0.0, 0.0
    for other in rids[1:]:
        diff = np.abs(np.stack([rows[(other, i)] for i in places]) - first)
        worst, mean = max(worst, float(diff.max())), max(mean, float(diff.mean()))
    return {"max_fraction": worst / scale, "mean_fraction": mean / scale, "scale": scale}


def whole_update(y: torch.Tensor) -> torch.Tensor:
    """The update that a mixer or feed-forward returned, as float32 rows: itself, or for float32 partial sums
    ``[parts, rows, width]`` (the rows of a larger decode step) their sum in order, as the next norm adds them."""
    if y.dim() == 2:
        return y.float()
    total = y[0].clone()
    for part in y[1:]:
        total += part
    return total


def random_sequence(vocab: int, n: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=gen).tolist()


# --- the cuttings ------------------------------------------------------------------------------

def cut_whole(trace: Trace, rid: str) -> None:
    trace.add_step([(rid, trace.remaining(rid), "all")], end=[rid])


def cut_tail_decode(trace: Trace, rid: str, tail: int = 32) -> None:
    n = trace.remaining(rid)
    trace.add_step([(rid, n - tail, "all")])
    for i in range(tail):
        trace.add_step([(rid, 1, "all")], end=[rid] if i == tail - 1 else [])


def cut_portions(trace: Trace, rid: str, sizes=(5, 2, 9, 3, 17, 2, 33, 4, 2, 11)) -> None:
    i = 0
    while trace.remaining(rid):
        n = min(sizes[i % len(sizes)], trace.remaining(rid))
        if trace.remaining(rid) - n == 1:   # never leave a lone token for a "portion": fold it in
            n += 1
        trace.add_step([(rid, n, "all")], end=[rid] if trace.remaining(rid) == n else [])
        i += 1


def cut_mixed(trace: Trace, rids: list[str], seed: int = 0, max_live: int = 4) -> None:
    """Up to ``max_live`` requests at a time: some feed portions of their prompt, others single
    tokens, some sit a step out; finished ones end and the next one starts in pages just freed."""
    rng = np.random.default_rng(seed)
    waiting = list(rids)
    live: dict[str, int] = {}          # request -> length of its "prompt" part (fed in portions)
    while waiting or live:
        while waiting and len(live) < max_live:
            rid = waiting.pop(0)
            total = len(trace.sequences[rid])
            live[rid] = max(2, int(total * rng.uniform(0.4, 0.8)))
        entries, ending = [], []
        for rid in list(live):
            if len(live) > 1 and rng.uniform() < 0.2:
                continue                # sits this step out
            fed, prompt = trace.fed(rid), live[rid]
            if fed < prompt:
                n = int(min(prompt - fed, rng.choice([2, 3, 7, 16, 21, 40])))
                if prompt - fed - n == 1:
                    n += 1
            else:
                n = 1
            n = min(n, trace.remaining(rid))
            entries.append((rid, n, "all"))
            if trace.remaining(rid) == n:
                ending.append(rid)
        if not entries:
            continue
        trace.add_step(entries, end=ending)
        for rid in ending:
            del live[rid]
