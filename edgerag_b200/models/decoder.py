"""A decoder assembled from a ``ModelPlan``: embedding, blocks run in the plan's order, norm, head.

The generic counterpart of ``EdgeRagDecoder.forward`` (edgerag/core/model.py:106-152).  Nothing in
this file knows an architecture: the plan names the parts, the registries build them, and the run
order is the plan's ``schedule`` list.  The model also derives what it needs from the cache (which
cache layers exist, how they group, which state records) and the full list of checkpoint tensors.
"""

from __future__ import annotations

import torch

from ..cache.manager import CacheLayout, KVGroupSpec, StateSpec
from ..ops import kernels
from ..parts.base import _REGISTRY, LayerCall, ModelPlan, Part, WeightSpec, build_part


class DecoderModel:
    def __init__(self, plan: ModelPlan, dtype: torch.dtype, device: torch.device) -> None:
        self.plan = plan
        self.dtype, self.device = dtype, device
        self.hidden_size, self.vocab_size = plan.hidden_size, plan.vocab_size
        self.embedding = build_part("embedding", plan.embedding, dtype, device)
        self.blocks = []
        #: (model-relative prefix, part) of everything that owns tensors
        self._owners: list[tuple[str, Part]] = [(plan.embedding.prefix, self.embedding)]
        for layer in plan.layers:
            norm1 = build_part("norm", layer.norm1, dtype, device)
            mixer = build_part("mixer", layer.mixer, dtype, device)
            norm2 = build_part("norm", layer.norm2, dtype, device)
            ffn = build_part("ffn", layer.ffn, dtype, device)
            try:
                block_cls = _REGISTRY["block"][layer.block.kind]
            except KeyError:
                raise KeyError(f"no block arrangement named {layer.block.kind!r}") from None
            block = block_cls(norm1=norm1, mixer=mixer, norm2=norm2, ffn=ffn, hidden=plan.hidden_size,
                              dtype=dtype, device=device, **layer.block.params)
            self.blocks.append(block)
            for spec, part in ((layer.norm1, norm1), (layer.mixer, mixer), (layer.norm2, norm2),
                               (layer.ffn, ffn), (layer.block, block)):
                self._owners.append((layer.prefix + spec.prefix, part))
        self.final_norm = build_part("norm", plan.final_norm, dtype, device) if plan.final_norm else None
        if self.final_norm is not None:
            self._owners.append((plan.final_norm.prefix, self.final_norm))
        self.head = build_part("head", plan.head, dtype, device)
        self._owners.append((plan.head.prefix, self.head))
        self.schedule: list[LayerCall] = list(plan.schedule)
        self.cache_layout = self._derive_cache_layout()
        #: every part may be captured in a CUDA graph (an attention mixer also vouches for its position encoding)
        self.graph_safe = all(part.graph_safe for _, part in self._owners) and all(
            getattr(getattr(b.mixer, "position", None), "graph_safe", True) for b in self.blocks)
        self.logits_stride = -(-plan.vocab_size // 8) * 8  # rows of the logits buffer start 32-byte aligned

    # --- cache needs ------------------------------------------------------------------------------

    def _derive_cache_layout(self) -> CacheLayout:
        n_cache_layers = 1 + max((c.cache_layer for c in self.schedule if c.cache_layer is not None), default=-1)
        owner: list[int | None] = [None] * n_cache_layers
        for call in self.schedule:
            if call.cache_layer is not None and call.writes_cache:
                if owner[call.cache_layer] is not None:
                    raise ValueError(f"cache layer {call.cache_layer} is written by two calls of the run order")
                owner[call.cache_layer] = call.layer
        layout = CacheLayout(placement=[None] * n_cache_layers)
        keys: list[tuple[int, int, int, int | None]] = []
        counts: list[int] = []
        for cl, layer in enumerate(owner):
            if layer is None:
                raise ValueError(f"cache layer {cl} is read but never written")
            spec = self.blocks[layer].mixer.cache_spec()
            if isinstance(spec, KVGroupSpec):
                key = (spec.n_kv_heads, spec.head_dim, spec.window, spec.v_head_dim)
                if key not in keys:
                    keys.append(key)
                    counts.append(0)
                g = keys.index(key)
                layout.placement[cl] = (g, counts[g])
                counts[g] += 1
            elif spec:
                for st in spec:
                    layout.states.append(StateSpec(f"{st.name}@{cl}", tuple(st.shape), st.dtype))
        layout.groups = [KVGroupSpec(c, *k) for k, c in zip(keys, counts)]
        return layout

    # --- weights ----------------------------------------------------------------------------------

    def weight_specs(self) -> list[WeightSpec]:
        """Every tensor of the checkpoint, with model-relative names."""
        specs, seen = [], set()
        for prefix, part in self._owners:
            for s in part.weight_specs():
                full = WeightSpec(prefix + s.name, s.shape, s.kind, s.fallback)
                if full.name not in seen:  # a layer built once owns its tensors once
                    seen.add(full.name)
                    specs.append(full)
        return specs

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        """Hand every part its tensors (``tensors`` has the names of ``weight_specs``)."""
        for prefix, part in self._owners:
            mine = {s.name: tensors[prefix + s.name] for s in part.weight_specs()}
            if mine:
                part.load_weights(mine)

    # --- one step ---------------------------------------------------------------------------------

    def forward(self, ctx) -> torch.Tensor | None:
        """Run the tokens of ``ctx`` through the stack; float32 logits ``[wanted, vocab]`` or None."""
        n = ctx.n_tokens
        hidden = ctx.buf("model.hidden", (n, self.hidden_size), torch.float32)
        self.embedding.forward(ctx, hidden)
        ctx.stream_written = kernels.launches()      # (the embedding wrote the residual stream: see the block)
        delta = None
        for call in self.schedule:
            before = ctx.stream_written
            delta = self.blocks[call.layer].forward(hidden, delta, ctx, call)
            if ctx.stream_written == before:      # a block that keeps no account of its writes to the stream:
                ctx.stream_written = float("inf")  # nobody may assume that the stream has settled
        w = ctx.n_wanted
        if w == 0:
            return None
        y = ctx.buf("model.final", (w, self.hidden_size), self.dtype)
        if self.final_norm is not None:
            self.final_norm.forward(hidden, y, delta, rows=ctx.want_rows, write_back=False,
                                    settled=kernels.launches() > ctx.stream_written)
        else:
            if delta is not None:
                kernels.residual_add(hidden, delta, self.dtype)
            kernels.gather_cast(hidden, y, ctx.want_rows)
        logits = ctx.buf("model.logits", (w, self.logits_stride), torch.float32)[:, : self.vocab_size]
        self.head.forward(y, logits)
        return logits
