"""Block arrangements: how a layer's norms, mixer and feed-forward are wired around the residual.

``PreNormBlock`` is the reference's ``DecoderLayer`` (edgerag/core/layers.py:366-374):
``h += mixer(norm1(h)); h += ffn(norm2(h))``.  Each residual add is fused into the norm that
follows it, so a block receives the previous block's update as ``delta`` and returns its own
feed-forward output as the update that is still to be added.
"""

from __future__ import annotations

import torch

from .base import Block, FeedForward, LayerCall, Mixer, Norm, register_part


@register_part("block", "prenorm")
class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward, hidden: int,
                 dtype: torch.dtype, device: torch.device) -> None:
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self.hidden = hidden
        self.dtype = dtype

    def forward(self, hidden: torch.Tensor, delta: torch.Tensor | None, ctx, call: LayerCall) -> torch.Tensor:
        n = hidden.shape[0]
        x = ctx.buf("block.normed", (n, self.hidden), self.dtype)
        self.norm1.forward(hidden, x, delta)          # hidden += delta; x = norm1(hidden)
        mixed = self.mixer.forward(x, ctx, call)
        self.norm2.forward(hidden, x, mixed)          # hidden += mixed; x = norm2(hidden)
        return self.ffn.forward(x, ctx)               # added by whichever norm comes next
