"""Interfaces and registries of the parts a decoder is put together from.

A model is data: a ``ModelPlan`` names, layer by layer, which norm, mixer, feed-forward and block
arrangement to build and with which sizes and constants, and in which order the layers run.  The
classes behind the names are looked up in the registries below, so a new kind of part is added by
registering a class (from anywhere, a test included) and naming it in a plan.  No part knows which
model it is in: it gets its sizes as constructor arguments and its tensors by name.

Interfaces (duck-typed; the base classes document them):

* every part: ``weight_specs() -> list[WeightSpec]`` (names relative to the part's prefix) and
  ``load_weights(tensors: dict[str, Tensor])`` with those relative names;
* ``Norm.forward(hidden, out, delta=None, rows=None, write_back=True)``;
* ``PositionEncoding.apply_and_store(qkv, ctx, n_q_heads, n_kv_heads, head_dim, pages, slots)`` and,
  optionally, ``project_apply_store(x, w_qkv, qkv, ctx, ...) -> bool`` (product, encoding and cache
  write in one kernel, where the part has one);
* ``Mixer.cache_spec()`` and ``Mixer.forward(x, ctx, call) -> Tensor``;
* ``FeedForward.forward(x, ctx) -> Tensor``;
* ``Block.forward(hidden, delta, ctx, call) -> delta`` (the update that is still to be added).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from ..cache.manager import KVGroupSpec, StateSpec


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part needs from the checkpoint.

    ``kind``: ``"matrix"`` is cast to the engine's element type (bfloat16 when serving);
    ``"vector32"`` is held in float32 whatever the file stores (norm weights: the value is kept,
    and a tensor stored in 32-bit stays 32-bit); ``"keep"`` keeps a 32-bit tensor as stored and
    casts 16-bit ones to the element type; ``"int"`` becomes int32.
    """

    name: str
    shape: tuple[int, ...]
    kind: str = "matrix"
    #: name (model-relative) of a tensor to share when this one is absent, e.g. a tied output head
    fallback: str | None = None


@dataclass
class PartSpec:
    """Which registered class to build and with which arguments."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    #: where the part's tensors live below its layer, e.g. ``"self_attn."``
    prefix: str = ""


@dataclass
class LayerSpec:
    """One layer: a block arrangement over a norm, a mixer, a second norm and a feed-forward."""

    prefix: str
    block: PartSpec
    norm1: PartSpec
    mixer: PartSpec
    norm2: PartSpec
    ffn: PartSpec


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: which layer runs and which cache layer it uses.

    A layer may appear in several calls (its weights are used again; each call then names a cache
    layer of its own), and a call with ``writes_cache=False`` reads the cache another call wrote.
    """

    layer: int
    cache_layer: int | None
    writes_cache: bool = True


@dataclass
class ModelPlan:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: list[LayerSpec]
    schedule: list[LayerCall]
    final_norm: PartSpec | None
    head: PartSpec
    #: prefixes under which a checkpoint may store the model-relative names, tried in order
    name_prefixes: tuple[str, ...] = ("model.text_model.", "model.", "")
    #: tensors of the checkpoint that belong to other towers and are not an error
    ignored_prefixes: tuple[str, ...] = ()


class Part:
    """Base of every part: owns tensors, knows their names, holds no reference to a model."""

    #: Whether ``forward`` may be captured in a CUDA graph and replayed for later steps of the same
    #: layout: everything that changes from step to step must then be read on the device from the
    #: step context's tensors (never baked in from its host copies), and nothing may allocate or
    #: synchronise.  Parts that do not say so keep their model on the eager path.
    graph_safe = False

    def weight_specs(self) -> list[WeightSpec]:
        return []

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        if tensors:
            raise ValueError(f"{type(self).__name__} takes no tensors")


class Norm(Part):
    def forward(self, hidden: torch.Tensor, out: torch.Tensor, delta: torch.Tensor | None = None,
                rows: torch.Tensor | None = None, write_back: bool = True, settled: bool = False) -> None:
        """``hidden`` (float32, the residual stream) gets ``delta`` added in place when given and
        ``write_back``; ``out`` receives the normed rows (all rows, or ``rows`` of them).  ``delta`` is
        ``[rows, hidden]`` of the model's element type or float32 partial sums ``[parts, rows, hidden]``.  ``settled`` is a
        hint that a norm may ignore: the caller vouches that ``hidden`` was not written by the kernel
        launched just before this call (only ``delta`` was), so it may be read while that kernel runs."""
        raise NotImplementedError


class PositionEncoding(Part):
    def apply_and_store(self, qkv: torch.Tensor, ctx: Any, n_q_heads: int, n_kv_heads: int, head_dim: int,
                        pages: tuple[torch.Tensor, torch.Tensor] | None, slots: torch.Tensor | None) -> None:
        """Encode positions into q and k of ``qkv`` (rows: q heads, k heads, v heads) and, when
        ``pages`` is given, write the encoded k and v to the tokens' cache slots."""
        raise NotImplementedError


    def project_apply_store(self, x: torch.Tensor, w_qkv: torch.Tensor, qkv: torch.Tensor, ctx: Any, n_q_heads: int,
                            n_kv_heads: int, head_dim: int, pages: tuple[torch.Tensor, torch.Tensor] | None,
                            slots: torch.Tensor | None) -> bool:
        """Optional: the product ``qkv = x @ w_qkv^T``, the encoding and the cache write as one
        kernel (only the q columns of ``qkv`` need to be valid afterwards).  Returns False, having
        done nothing, when the part has no such kernel for these operands; the mixer then makes the
        product itself and calls ``apply_and_store``."""
        return False


class Mixer(Part):
    def cache_spec(self) -> KVGroupSpec | list[StateSpec] | None:
        """What one call of this mixer keeps between steps: paged keys/values (``n_layers`` is
        ignored), state records of fixed size, or nothing."""
        return None

    def forward(self, x: torch.Tensor, ctx: Any, call: LayerCall) -> torch.Tensor:
        """The update of the residual stream for the normed rows ``x``: ``[rows, hidden]`` of the model's
        element type, or float32 partial sums ``[parts, rows, hidden]`` whose sum in order is the update
        (a norm adds them as it reads)."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
        """As ``Mixer.forward``: the update, whole or as float32 partial sums."""
        raise NotImplementedError


class Block(Part):
    def forward(self, hidden: torch.Tensor, delta: torch.Tensor | None, ctx: Any, call: LayerCall) -> torch.Tensor | None:
        raise NotImplementedError


# --- registries -------------------------------------------------------------------------------

CATEGORIES = ("norm", "position", "mixer", "ffn", "block", "embedding", "head")
_REGISTRY: dict[str, dict[str, Callable[..., Part]]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str) -> Callable:
    """Class decorator: ``@register_part("mixer", "attention")``."""
    if category not in _REGISTRY:
        raise KeyError(f"unknown part category {category!r}; have {CATEGORIES}")

    def deco(cls):
        _REGISTRY[category][kind] = cls
        return cls

    return deco


def build_part(category: str, spec: PartSpec, dtype: torch.dtype, device: torch.device) -> Part:
    """Instantiate the class registered for ``spec.kind`` with ``spec.params`` plus dtype and device."""
    try:
        cls = _REGISTRY[category][spec.kind]
    except KeyError:
        raise KeyError(f"no {category} part named {spec.kind!r}; registered: {sorted(_REGISTRY[category])}") from None
    return cls(**spec.params, dtype=dtype, device=device)


def registered(category: str) -> list[str]:
    return sorted(_REGISTRY[category])
