"""Input and output ends of the decoder.

``TokenEmbedding``: a plain table lookup without scale, or rows of caller-given embeddings
(edgerag/core/model.py:106-110: exactly one of ids and embeddings per token); the result is
written to the float32 residual stream.  ``LMHead``: bias-free projection to float32 logits over
the rows that were asked for (edgerag/core/model.py:150-152); a checkpoint without
``lm_head.weight`` whose config ties the embeddings shares the table.
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

    def __init__(self, vocab: int, hidden: int, tied: bool, dtype: torch.dtype, device: torch.device) -> None:
        self.vocab, self.hidden, self.tied = vocab, hidden, tied
        self.dtype, self.device = dtype, device
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec("weight", (self.vocab, self.hidden),
                           fallback="embed_tokens.weight" if self.tied else None)]

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].to(device=self.device, dtype=self.dtype).contiguous()

    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> None:
        kernels.linear(x, self.weight, logits)
