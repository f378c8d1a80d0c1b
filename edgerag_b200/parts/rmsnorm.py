"""RMSNorm with the residual add fused in.

The reference's formula (edgerag/core/layers.py:40-47): statistics in float32, the normalised
value cast back to the model's element type, then the weight multiply.  Here the residual stream
itself stays in float32, so the sum ``hidden + delta`` that the reference forms in 16-bit
(edgerag/core/layers.py:372-373) is exact to float32.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import Norm, WeightSpec, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, size: int, eps: float, dtype: torch.dtype, device: torch.device) -> None:
        self.size = size
        self.eps = float(eps)
        self.dtype = dtype
        self.device = device
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec("weight", (self.size,), kind="vector32")]

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].to(device=self.device, dtype=torch.float32).contiguous()

    def forward(self, hidden, out, delta=None, rows=None, write_back=True, settled=False) -> None:
        kernels.add_rmsnorm(hidden, self.weight, out, self.eps, delta=delta, rows=rows, write_back=write_back, settled=settled)
