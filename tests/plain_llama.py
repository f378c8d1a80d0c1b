"""Plain, slow implementation of the SmolVLM Llama decoder: the oracle of the test suite.

Whole sequences, no cache, no batching tricks, one function per part, PyTorch on the CPU (or
wherever the tensors live).  It shares no code with ``edgerag_b200``: it reads ``config.json`` as
a plain dict and the weights as a plain ``name -> tensor`` dict in the checkpoint's own names.

Every function is written from the formulas of Tejas544/edgerag and cites the file and lines
(paths inside that project).  ``tests/golden/make_golden.py`` compared this file once with the
project's own ``EdgeRagDecoder`` on tiny random models; the outputs it wrote are committed in
``tests/golden/`` and ``tests/test_plain.py`` checks this file against them.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# --------------------------------------------------------------------------------------------
# configuration (edgerag/core/spec.py:195-234)
# --------------------------------------------------------------------------------------------

def read_config(folder: str | Path) -> dict:
    """config.json as the flat dict of decoder sizes the functions below take.

    Mirrors ``ModelSpec.from_hf_config`` (edgerag/core/spec.py:206-234): sizes come from
    ``text_config`` when the file is a composite, ``num_key_value_heads`` defaults to the number
    of query heads, ``head_dim`` to ``hidden_size // heads``, and ``rope_theta`` is looked up in
    ``rope_parameters`` first and never defaulted (edgerag/core/spec.py:39-63).
    """
    raw = json.loads((Path(folder) / "config.json").read_text())
    txt = raw.get("text_config", raw)
    heads = txt["num_attention_heads"]
    rope = txt.get("rope_parameters") or {}
    theta = rope.get("rope_theta", txt.get("rope_theta"))
    if theta is None:
        raise ValueError("rope_theta missing")
    return {
        "n_layers": txt["num_hidden_layers"],
        "hidden": txt["hidden_size"],
        "n_q": heads,
        "n_kv": txt.get("num_key_value_heads") or heads,
        "head_dim": txt.get("head_dim") or txt["hidden_size"] // heads,
        "vocab": txt["vocab_size"],
        "theta": float(theta),
        "eps": float(txt["rms_norm_eps"]),
        "inter": txt["intermediate_size"],
        "tied": bool(txt.get("tie_word_embeddings", raw.get("tie_word_embeddings", False))),
    }


def read_weights(folder: str | Path, dtype: torch.dtype = torch.float32) -> dict[str, torch.Tensor]:
    """All tensors of model.safetensors by name, cast to ``dtype`` (floating ones only)."""
    from safetensors.torch import load_file

    tensors = load_file(str(Path(folder) / "model.safetensors"))
    return {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}


def _w(weights: dict[str, torch.Tensor], name: str) -> torch.Tensor:
    """Look a tensor up under the prefixes a checkpoint may carry (edgerag/core/model.py:274-295)."""
    for prefix in ("model.text_model.", "model.", ""):
        if prefix + name in weights:
            return weights[prefix + name]
    raise KeyError(name)


# --------------------------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------------------------

def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """edgerag/core/layers.py:40-47: statistics in fp32, cast back, then the weight multiply."""
    dtype = x.dtype
    x32 = x.to(torch.float32)
    variance = x32.pow(2).mean(-1, keepdim=True)
    x32 = x32 * torch.rsqrt(variance + eps)
    return weight * x32.to(dtype)


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """edgerag/core/layers.py:66-90: fp32 cos and sin of shape ``(n, head_dim)``.

    ``inv_freq[j] = 1 / theta**(2j / head_dim)``; the angle table is the outer product with the
    logical positions, repeated twice along the last axis (halves convention).
    """
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    freqs = positions.to(torch.float32)[:, None] * inv_freq[None, :].to(positions.device)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """edgerag/core/layers.py:93-101: ``[-x2, x1]`` over the two halves of the last axis."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """edgerag/core/layers.py:104-114 for one tensor ``(heads, n, head_dim)``; cos/sin ``(n, head_dim)``."""
    return x * cos[None].to(x.dtype) + rotate_half(x) * sin[None].to(x.dtype)


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """edgerag/core/layers.py:117-134: each kv head repeated ``n_rep`` times consecutively."""
    return x if n_rep == 1 else x.repeat_interleave(n_rep, dim=0)


def causal_mask(n: int, dtype: torch.dtype, device, window: int | None = None) -> torch.Tensor:
    """edgerag/core/layers.py:243-254 with no past: 0 where ``k <= q`` else ``finfo.min``.

    ``window`` (not in the reference: it has no windowed layer) additionally hides keys with
    ``k <= q - window``; it exists for the tests of the engine's windowed-cache machinery.
    """
    q = torch.arange(n, device=device)[:, None]
    k = torch.arange(n, device=device)[None, :]
    keep = k <= q
    if window is not None:
        keep &= k > q - window
    return torch.where(keep, 0.0, torch.finfo(dtype).min).to(dtype)


def attention_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                   window: int | None = None) -> torch.Tensor:
    """edgerag/core/layers.py:212-224 (eager): q ``(nq, n, D)``, k/v ``(nkv, n, D)`` -> ``(n, nq*D)``."""
    n_rep = q.shape[0] // k.shape[0]
    k = repeat_kv(k, n_rep)
    v = repeat_kv(v, n_rep)
    scores = torch.matmul(q, k.transpose(1, 2)) * scale
    scores = scores + causal_mask(q.shape[1], q.dtype, q.device, window)[None]
    probs = torch.softmax(scores, dim=-1, dtype=torch.float32).to(q.dtype)
    out = torch.matmul(probs, v)                       # (nq, n, D)
    return out.transpose(0, 1).reshape(q.shape[1], -1)


def attention(x: torch.Tensor, positions: torch.Tensor, wq, wk, wv, wo, cfg: dict,
              window: int | None = None) -> torch.Tensor:
    """edgerag/core/layers.py:294-322: projections, RoPE on q and k, causal GQA attention, o_proj."""
    n, d = x.shape[0], cfg["head_dim"]
    q = (x @ wq.T).view(n, cfg["n_q"], d).transpose(0, 1)
    k = (x @ wk.T).view(n, cfg["n_kv"], d).transpose(0, 1)
    v = (x @ wv.T).view(n, cfg["n_kv"], d).transpose(0, 1)
    cos, sin = rope_tables(positions, d, cfg["theta"])
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    return attention_core(q, k, v, d ** -0.5, window) @ wo.T


def swiglu(x: torch.Tensor, wg, wu, wd) -> torch.Tensor:
    """edgerag/core/layers.py:341: ``down(silu(gate(x)) * up(x))``."""
    return (torch.nn.functional.silu(x @ wg.T) * (x @ wu.T)) @ wd.T


def decoder_layer(h: torch.Tensor, positions: torch.Tensor, weights: dict, i: int, cfg: dict) -> torch.Tensor:
    """edgerag/core/layers.py:366-374: pre-norm block with two residuals."""
    p = f"layers.{i}."
    x = rms_norm(h, _w(weights, p + "input_layernorm.weight"), cfg["eps"])
    h = h + attention(
        x, positions,
        _w(weights, p + "self_attn.q_proj.weight"), _w(weights, p + "self_attn.k_proj.weight"),
        _w(weights, p + "self_attn.v_proj.weight"), _w(weights, p + "self_attn.o_proj.weight"), cfg,
    )
    y = rms_norm(h, _w(weights, p + "post_attention_layernorm.weight"), cfg["eps"])
    return h + swiglu(
        y, _w(weights, p + "mlp.gate_proj.weight"), _w(weights, p + "mlp.up_proj.weight"),
        _w(weights, p + "mlp.down_proj.weight"),
    )


def lm_head_weight(weights: dict, cfg: dict) -> torch.Tensor:
    """edgerag/core/model.py:281-283 fills lm_head from the checkpoint; tied checkpoints share the table."""
    if "lm_head.weight" in weights:
        return weights["lm_head.weight"]
    if not cfg["tied"]:
        raise KeyError("lm_head.weight")
    return _w(weights, "embed_tokens.weight")


def embed(weights: dict, token_ids: torch.Tensor) -> torch.Tensor:
    """edgerag/core/model.py:109: a plain table lookup, no scale."""
    return _w(weights, "embed_tokens.weight")[token_ids]


def forward(weights: dict, cfg: dict, token_ids=None, embeds: torch.Tensor | None = None) -> torch.Tensor:
    """edgerag/core/model.py:106-152 for one whole sequence: logits ``(n, vocab)`` at every position.

    Exactly one of ``token_ids`` (list or 1-D tensor) and ``embeds`` ``(n, hidden)``.
    """
    if (token_ids is None) == (embeds is None):
        raise ValueError("pass exactly one of token_ids or embeds")
    if embeds is None:
        h = embed(weights, torch.as_tensor(token_ids, dtype=torch.long))
    else:
        h = embeds.to(_w(weights, "norm.weight").dtype)
    positions = torch.arange(h.shape[0], device=h.device)
    for i in range(cfg["n_layers"]):
        h = decoder_layer(h, positions, weights, i, cfg)
    h = rms_norm(h, _w(weights, "norm.weight"), cfg["eps"])
    return h @ lm_head_weight(weights, cfg).T


# --------------------------------------------------------------------------------------------
# generation (edgerag/serve/executor.py:131-154, bench/pipeline.py:100-110)
# --------------------------------------------------------------------------------------------

def greedy_generate(weights: dict, cfg: dict, prompt: list[int], n_new: int,
                    eos: int | None = None) -> list[int]:
    """Greedy argmax, the whole sequence recomputed for every token (no cache)."""
    seq, out = list(prompt), []
    for _ in range(n_new):
        token = int(forward(weights, cfg, seq)[-1].argmax())
        out.append(token)
        seq.append(token)
        if eos is not None and token == eos:
            break
    return out


def temperature_probs(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """``softmax(logits / T)`` in float64: the distribution the engine's sampler must draw from.

    The reference samples greedily only (edgerag/serve/app.py:105-120 refuses anything else), so
    this is the textbook formula rather than a citation.
    """
    return torch.softmax(logits.to(torch.float64) / temperature, dim=-1)


def inverse_cdf_pick(probs: torch.Tensor, u: float) -> int:
    """First index whose cumulative probability exceeds ``u`` (float64)."""
    cdf = torch.cumsum(probs.to(torch.float64), dim=-1)
    idx = int(torch.searchsorted(cdf, torch.tensor(u, dtype=torch.float64), right=True))
    return min(idx, probs.numel() - 1)


# --------------------------------------------------------------------------------------------
# the two tiny configurations of the suite; they differ in every size and option
# --------------------------------------------------------------------------------------------

TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 160, "vocab_size": 512, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 256,
    "hidden_act": "silu", "pad_token_id": 0,
}

TINY_B = {
    "architectures": ["SmolVLMForConditionalGeneration"], "model_type": "smolvlm",
    "text_config": {
        "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
        "head_dim": 32, "intermediate_size": 256, "vocab_size": 1000,
        "rope_parameters": {"rope_theta": 100000.0, "rope_type": "default"},
        "rms_norm_eps": 1e-6, "max_position_embeddings": 512, "hidden_act": "silu", "pad_token_id": 2,
    },
    "tie_word_embeddings": False,
}


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    """Names and shapes of every tensor of a checkpoint (edgerag/core/model.py:274-295)."""
    h, d = cfg["hidden"], cfg["head_dim"]
    shapes = {"model.embed_tokens.weight": (cfg["vocab"], h), "model.norm.weight": (h,)}
    for i in range(cfg["n_layers"]):
        p = f"model.layers.{i}."
        shapes[p + "self_attn.q_proj.weight"] = (cfg["n_q"] * d, h)
        shapes[p + "self_attn.k_proj.weight"] = (cfg["n_kv"] * d, h)
        shapes[p + "self_attn.v_proj.weight"] = (cfg["n_kv"] * d, h)
        shapes[p + "self_attn.o_proj.weight"] = (h, cfg["n_q"] * d)
        shapes[p + "mlp.gate_proj.weight"] = (cfg["inter"], h)
        shapes[p + "mlp.up_proj.weight"] = (cfg["inter"], h)
        shapes[p + "mlp.down_proj.weight"] = (h, cfg["inter"])
        shapes[p + "input_layernorm.weight"] = (h,)
        shapes[p + "post_attention_layernorm.weight"] = (h,)
    if not cfg["tied"]:
        shapes["lm_head.weight"] = (cfg["vocab"], h)
    return shapes


def write_model_folder(folder: str | Path, raw_config: dict, seed: int, std: float = 0.02,
                       norm_jitter: float = 0.1, dtype: torch.dtype = torch.float32) -> Path:
    """Write config.json and model.safetensors with seeded random weights, independently of the product.

    Matrices are ``N(0, std)``; norm weights are ``1 + norm_jitter * N(0, 1)`` so that a norm
    weight that is dropped or applied in the wrong place shows.
    """
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(raw_config, indent=1))
    cfg = read_config(folder)
    gen = torch.Generator().manual_seed(seed)
    tensors = {}
    for name, shape in tensor_shapes(cfg).items():
        if len(shape) == 1:
            t = 1.0 + norm_jitter * torch.randn(shape, generator=gen)
        else:
            t = std * torch.randn(shape, generator=gen)
        tensors[name] = t.to(dtype).contiguous()
    save_file(tensors, str(folder / "model.safetensors"))
    return folder


def flops_per_token(cfg: dict) -> float:  # pragma: no cover - a convenience for notes
    """Linear-layer flops of one token (2 per multiply-add), without attention."""
    h, d = cfg["hidden"], cfg["head_dim"]
    per_layer = 2 * h * d * (cfg["n_q"] + 2 * cfg["n_kv"]) + 2 * h * d * cfg["n_q"] + 6 * h * cfg["inter"]
    return cfg["n_layers"] * per_layer + 2 * h * cfg["vocab"]


__all__ = [n for n in dir() if not n.startswith("_") and n not in ("json", "math", "Path", "torch")]
