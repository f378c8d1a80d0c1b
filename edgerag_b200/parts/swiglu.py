"""The gated feed-forward of the Llama decoder: ``down(silu(gate(x)) * up(x))``, no biases
(edgerag/core/layers.py:332-341).  ``gate`` and ``up`` are stored as one matrix ``[Wg; Wu]`` so a
single product feeds the gate kernel, which computes ``silu(g) * u`` in float32 and rounds once; for
the few rows of a decode step the product and the gate are one kernel with the same result.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import FeedForward, WeightSpec, register_part


@register_part("ffn", "swiglu")
class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, hidden: int, intermediate: int, dtype: torch.dtype, device: torch.device) -> None:
        self.hidden, self.intermediate = hidden, intermediate
        self.dtype, self.device = dtype, device
        self.w_gate_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec("gate_proj.weight", (self.intermediate, self.hidden)),
                WeightSpec("up_proj.weight", (self.intermediate, self.hidden)),
                WeightSpec("down_proj.weight", (self.hidden, self.intermediate))]

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        cast = lambda t: t.to(device=self.device, dtype=self.dtype)  # noqa: E731
        self.w_gate_up = torch.cat([cast(tensors["gate_proj.weight"]), cast(tensors["up_proj.weight"])], 0).contiguous()
        self.w_down = cast(tensors["down_proj.weight"]).contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        n = x.shape[0]
        act = ctx.buf("ffn.act", (n, self.intermediate), self.dtype)
        if kernels.linear_glu_supported(x, self.w_gate_up):
            kernels.linear_glu(x, self.w_gate_up, act)       # a few rows: product and gate in one kernel
        else:
            gate_up = ctx.buf("ffn.gate_up", (n, 2 * self.intermediate), self.dtype)
            kernels.linear(x, self.w_gate_up, gate_up)
            kernels.swiglu(gate_up, act)
        n_parts = kernels.linear_parts_count(act, self.w_down)
        if n_parts:      # the rows of a larger decode step: k split over the SMs, the norm after adds the parts
            y = ctx.buf("ffn.out_parts", (n_parts, n, self.hidden), torch.float32)
            kernels.linear_parts(act, self.w_down, y)
            return y
        y = ctx.buf("ffn.out", (n, self.hidden), self.dtype)
        kernels.linear(act, self.w_down, y)
        return y
