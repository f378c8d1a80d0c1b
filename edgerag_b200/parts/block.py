"""Block arrangements: how a layer's norms, mixer and feed-forward are wired around the residual.

``PreNormBlock`` is the reference's ``DecoderLayer`` (edgerag/core/layers.py:366-374):
``h += mixer(norm1(h)); h += ffn(norm2(h))``.  Each residual add is fused into the norm that
follows it, so a block receives the previous block's update as ``delta`` and returns its own
feed-forward output as the update that is still to be added.
"""

from __future__ import annotations

import torch

from ..ops import kernels
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
        # A norm may read the stream while the kernel before it still runs if that kernel did not write the
        # stream: true when at least one kernel of this package has been launched since the stream's last
        # writer (`ctx.stream_written`, the launch count right after it).
        settled = lambda: kernels.launches() > getattr(ctx, "stream_written", float("inf"))   # noqa: E731
        self.norm1.forward(hidden, x, delta, settled=settled())   # hidden += delta; x = norm1(hidden)
        if delta is not None:
            ctx.stream_written = kernels.launches()
        mixed = self.mixer.forward(x, ctx, call)
        self.norm2.forward(hidden, x, mixed, settled=settled())   # hidden += mixed; x = norm2(hidden)
        ctx.stream_written = kernels.launches()
        return self.ffn.forward(x, ctx)               # added by whichever norm comes next
