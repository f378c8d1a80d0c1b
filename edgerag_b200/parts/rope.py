"""Position encodings that act on queries and keys before the keys are cached.

``RotaryHalves`` is the reference's RoPE (edgerag/core/layers.py:63-114): ``inv_freq[j] =
1 / theta**(2j / D)`` built exactly as there (int64 arange, float32 division and power), angles
``position * inv_freq`` in float32, and the halves convention ``[-x2, x1]``.  The rotation runs in
the same kernel that writes keys and values to their cache slots, so the cache holds rotated keys
(edgerag/core/layers.py:301-306) and a key's encoding depends on its own logical position only.

``NoPosition`` encodes nothing and only writes the cache; it is what a mixer uses when another
part has already put positions into the stream.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import PositionEncoding, register_part


@register_part("position", "rope_halves")
class RotaryHalves(PositionEncoding):
    graph_safe = True

    def __init__(self, head_dim: int, theta: float, dtype: torch.dtype, device: torch.device,
                 rot_dim: int | None = None) -> None:
        self.head_dim = head_dim
        self.rot_dim = head_dim if rot_dim is None else rot_dim
        if self.rot_dim % 2 or not 0 < self.rot_dim <= head_dim:
            raise ValueError(f"rot_dim {self.rot_dim} must be even and at most head_dim {head_dim}")
        self.theta = float(theta)
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.rot_dim, 2, dtype=torch.int64).float() / self.rot_dim))
        self.inv_freq = inv_freq.to(device=device, dtype=torch.float32).contiguous()

    def apply_and_store(self, qkv, ctx, n_q_heads, n_kv_heads, head_dim, pages, slots) -> None:
        k_pages, v_pages = pages if pages is not None else (None, None)
        kernels.rope_cache_write(
            qkv, ctx.positions, self.inv_freq, n_q_heads, n_kv_heads, head_dim, self.rot_dim,
            slots=slots, k_pages=k_pages, v_pages=v_pages, page_size=ctx.page_size)

    def project_apply_store(self, x, w_qkv, qkv, ctx, n_q_heads, n_kv_heads, head_dim, pages, slots) -> bool:
        """A few rows (a decode step): the rotation and the cache write ride in the product's epilogue."""
        if pages is None or slots is None or not kernels.linear_rope_store_supported(x, w_qkv, head_dim, self.rot_dim):
            return False
        kernels.linear_rope_store(x, w_qkv, qkv, ctx.positions, self.inv_freq, n_q_heads, n_kv_heads, head_dim,
                                  slots, pages[0], pages[1], ctx.page_size)
        return True


@register_part("position", "none")
class NoPosition(PositionEncoding):
    graph_safe = True

    def __init__(self, dtype: torch.dtype, device: torch.device, **_unused) -> None:
        pass

    def apply_and_store(self, qkv, ctx, n_q_heads, n_kv_heads, head_dim, pages, slots) -> None:
        if pages is None:
            return
        kernels.rope_cache_write(qkv, ctx.positions, None, n_q_heads, n_kv_heads, head_dim, 0,
                                 slots=slots, k_pages=pages[0], v_pages=pages[1], page_size=ctx.page_size)
