"""Input and output ends of the decoder.

``TokenEmbedding``: a plain table lookup without scale, or rows of caller-given embeddings
(edgerag/core/model.py:106-110: exactly one of ids and embeddings per token); the result is
written to the float32 residual stream.  ``LMHead``: bias-free projection to float32 logits over
the rows that were asked for (edgerag/core/model.py:150-152); where the plan names a tensor to
tie the head to, a checkpoint without a head of its own shares that tensor.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import Part, WeightSpec, register_part


@register_part("embedding", "table")
class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab: int, hidden: int, dtype: torch.dtype, device: torch.device) -> None:
        self.vocab, self.hidden = vocab, hidden
        self.dtype, self.device = dtype, device
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec("weight", (self.vocab, self.hidden))]

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].to(device=self.device, dtype=self.dtype).contiguous()

    def forward(self, ctx, hidden: torch.Tensor) -> None:
        kernels.embed_rows(hidden, self.weight, ctx.token_ids, ctx.status, embeds=ctx.embeds,
                           embed_row=ctx.embed_row if ctx.embeds is not None else None)


@register_part("head", "linear")
class LMHead(Part):
    graph_safe = True

    def __init__(self, vocab: int, hidden: int, dtype: torch.dtype, device: torch.device,
                 tied_to: str | None = None) -> None:
        """``tied_to``: model-relative name of the tensor to share when the checkpoint has no head of
        its own (the plan names it; this part does not know what the model calls its embedding)."""
        self.vocab, self.hidden, self.tied_to = vocab, hidden, tied_to
        self.dtype, self.device = dtype, device
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec("weight", (self.vocab, self.hidden), fallback=self.tied_to)]

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].to(device=self.device, dtype=self.dtype).contiguous()

    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> None:
        kernels.linear(x, self.weight, logits)
