"""Typed configuration of the SmolVLM / Llama text decoder, read from the checkpoint's config.json.

The counterpart of ``ModelSpec`` (edgerag/core/spec.py:66-134) and of its constructor
``ModelSpec.from_hf_config`` (edgerag/core/spec.py:195-234), with two differences: the file is read
directly as JSON (no library config class), and only the decoder's fields are kept.  Every size
and constant the layers use comes from here; nothing is assumed in code.

Keys read (from ``text_config`` when the file is a SmolVLM composite, else from the top level):
``num_hidden_layers, hidden_size, num_attention_heads, num_key_value_heads, head_dim, vocab_size,
max_position_embeddings, rope_parameters.rope_theta | rope_theta, pad_token_id, rms_norm_eps,
intermediate_size, hidden_act, tie_word_embeddings``; from the top level ``architectures`` and
``model_type``.  Keys that would change the arithmetic and are not implemented are refused by name:
``rope_scaling`` / ``rope_parameters.rope_type`` other than default, ``partial_rotary_factor``,
``attention_bias``, ``mlp_bias``, ``sliding_window``, logit soft-capping.
"""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """config.json is missing a key, or holds a value the decoder cannot run with."""


def _rope_theta(txt: dict[str, Any], where: str) -> float:
    """RoPE base, never defaulted: a wrong base runs and is silently wrong (edgerag/core/spec.py:39-63)."""
    params = txt.get("rope_parameters")
    if isinstance(params, dict) and params.get("rope_theta") is not None:
        return float(params["rope_theta"])
    if txt.get("rope_theta") is not None:
        return float(txt["rope_theta"])
    raise ConfigError(
        f"{where}: rope_theta is neither in rope_parameters nor a key of its own; refusing to default it"
    )


def _refuse_what_is_not_built(txt: dict[str, Any], where: str) -> None:
    """Options of Llama-style configurations that change the arithmetic and that this decoder does not
    implement (the reference has none of them either: edgerag/core/layers.py:63-90 has one rotary
    formula, edgerag/core/layers.py:280-283,336-338 build every projection without bias, and
    edgerag/core/layers.py:243-254 masks causally without a window).  A model that sets one of them
    would load and run with wrong logits, so it is refused by the key's name."""
    scaling = txt.get("rope_scaling")
    if scaling is not None:
        kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, dict) else scaling
        if kind not in (None, "default"):
            raise ConfigError(f"{where}: rope_scaling of type {kind!r} is not supported (plain rotary angles only)")
    params = txt.get("rope_parameters")
    if isinstance(params, dict):
        kind = params.get("rope_type", params.get("type"))
        if kind not in (None, "default"):
            raise ConfigError(f"{where}: rope_parameters.rope_type {kind!r} is not supported (plain rotary angles only)")
        factor = params.get("factor")
        if factor not in (None, 1, 1.0):
            raise ConfigError(f"{where}: rope_parameters.factor {factor!r} is not supported")
        partial = params.get("partial_rotary_factor")
        if partial not in (None, 1, 1.0):
            raise ConfigError(f"{where}: rope_parameters.partial_rotary_factor {partial!r} is not supported")
    if txt.get("partial_rotary_factor") not in (None, 1, 1.0):
        raise ConfigError(f"{where}: partial_rotary_factor {txt['partial_rotary_factor']!r} is not supported")
    for key in ("attention_bias", "mlp_bias"):
        if txt.get(key):
            raise ConfigError(f"{where}: {key} is set; projections with a bias are not supported")
    if txt.get("use_sliding_window") or (txt.get("sliding_window") and txt.get("use_sliding_window") is not False):
        raise ConfigError(f"{where}: sliding_window is set; this architecture attends to every earlier token")
    for key in ("attn_logit_softcapping", "final_logit_softcapping"):
        if txt.get(key):
            raise ConfigError(f"{where}: {key} is set; logit soft-capping is not supported")


def _need(txt: dict[str, Any], key: str, where: str) -> Any:
    if txt.get(key) is None:
        raise ConfigError(f"{where}: config.json has no '{key}'")
    return txt[key]


@dataclass(frozen=True)
class DecoderConfig:
    """Sizes and constants of one dense pre-norm decoder (RMSNorm, GQA + RoPE, SwiGLU)."""

    architecture: str
    n_layers: int
    hidden_size: int
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float
    rms_norm_eps: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    hidden_act: str = "silu"
    pad_token_id: int = 0

    def __post_init__(self) -> None:
        for name in ("n_layers", "hidden_size", "n_q_heads", "n_kv_heads", "head_dim",
                     "intermediate_size", "vocab_size", "max_position_embeddings"):
            if int(getattr(self, name)) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.n_q_heads % self.n_kv_heads:
            # edgerag/core/spec.py:126-134
            raise ConfigError(
                f"{self.n_q_heads} query heads are not divisible by {self.n_kv_heads} key/value heads"
            )
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} is odd: rotary halves need an even size")
        if not 0 <= self.pad_token_id < self.vocab_size:
            # edgerag/core/spec.py:111-120
            raise ConfigError(f"pad_token_id {self.pad_token_id} is outside vocab_size {self.vocab_size}")
        if self.hidden_act != "silu":
            # edgerag/core/layers.py:334-335
            raise ConfigError(f"unsupported activation {self.hidden_act!r}; expected silu")
        if not (self.rms_norm_eps > 0 and self.rope_theta > 0):
            raise ConfigError("rms_norm_eps and rope_theta must be positive")

    # --- derived (edgerag/core/spec.py:122-143) -------------------------------------------------

    @property
    def n_rep(self) -> int:
        """Query heads per key/value head; 1 is plain multi-head attention."""
        return self.n_q_heads // self.n_kv_heads

    @property
    def uses_gqa(self) -> bool:
        return self.n_kv_heads < self.n_q_heads

    def kv_bytes_per_token(self, itemsize: int = 2) -> int:
        """Bytes of cache one token occupies over all layers (edgerag/core/spec.py:138-143)."""
        return 2 * self.n_layers * self.n_kv_heads * self.head_dim * itemsize

    def n_parameters(self) -> int:
        h, d = self.hidden_size, self.head_dim
        per_layer = h * d * (2 * self.n_q_heads + 2 * self.n_kv_heads) + 3 * h * self.intermediate_size + 2 * h
        head = 0 if self.tie_word_embeddings else self.vocab_size * h
        return self.n_layers * per_layer + self.vocab_size * h + h + head

    # --- construction ---------------------------------------------------------------------------

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str = "config") -> "DecoderConfig":
        txt = raw.get("text_config", raw)
        if not isinstance(txt, dict):
            raise ConfigError(f"{where}: text_config is not an object")
        archs = raw.get("architectures") or []
        architecture = archs[0] if archs else raw.get("model_type")
        if not architecture:
            raise ConfigError(f"{where}: neither 'architectures' nor 'model_type' names the model")
        _refuse_what_is_not_built(txt, where)
        heads = int(_need(txt, "num_attention_heads", where))
        hidden = int(_need(txt, "hidden_size", where))
        tie = txt.get("tie_word_embeddings", raw.get("tie_word_embeddings", False))
        return cls(
            architecture=str(architecture),
            n_layers=int(_need(txt, "num_hidden_layers", where)),
            hidden_size=hidden,
            n_q_heads=heads,
            n_kv_heads=int(txt.get("num_key_value_heads") or heads),
            head_dim=int(txt.get("head_dim") or hidden // heads),
            intermediate_size=int(_need(txt, "intermediate_size", where)),
            vocab_size=int(_need(txt, "vocab_size", where)),
            rope_theta=_rope_theta(txt, where),
            rms_norm_eps=float(_need(txt, "rms_norm_eps", where)),
            max_position_embeddings=int(txt.get("max_position_embeddings") or 8192),
            tie_word_embeddings=bool(tie),
            hidden_act=str(txt.get("hidden_act", "silu")),
            pad_token_id=int(txt.get("pad_token_id") or 0),
        )

    @classmethod
    def from_json(cls, path: str | Path) -> "DecoderConfig":
        """Read ``path`` (a config.json, or the folder that holds one)."""
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        if not path.is_file():
            raise ConfigError(f"{path} does not exist")
        try:
            raw = json.loads(path.read_text())
        except json.JSONDecodeError as exc:
            raise ConfigError(f"{path}: not valid JSON ({exc})") from exc
        return cls.from_dict(raw, str(path))

    def to_hf_dict(self) -> dict[str, Any]:
        """A flat Llama-style config.json that ``from_dict`` reads back to an equal object."""
        return {
            "architectures": [self.architecture],
            "model_type": "llama",
            "num_hidden_layers": self.n_layers,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.n_q_heads,
            "num_key_value_heads": self.n_kv_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "pad_token_id": self.pad_token_id,
        }

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)
