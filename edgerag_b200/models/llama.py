"""The SmolVLM / Llama text decoder as a plan of parts.

Layer structure of ``EdgeRagDecoder`` (edgerag/core/model.py:61-70) and ``DecoderLayer``
(edgerag/core/layers.py:354-374): every layer is a pre-norm block of RMSNorm, grouped-query
attention with rotary halves, RMSNorm, SwiGLU; a final RMSNorm; a bias-free head.  Tensor names are
those the reference copies from (edgerag/core/model.py:274-295).
"""

from __future__ import annotations

from ..config.model_config import DecoderConfig
from ..parts.base import LayerCall, LayerSpec, ModelPlan, PartSpec


def llama_plan(cfg: DecoderConfig) -> ModelPlan:
    h = cfg.hidden_size
    norm = lambda prefix: PartSpec("rmsnorm", {"size": h, "eps": cfg.rms_norm_eps}, prefix)  # noqa: E731
    layers = []
    for i in range(cfg.n_layers):
        layers.append(LayerSpec(
            prefix=f"layers.{i}.",
            block=PartSpec("prenorm"),
            norm1=norm("input_layernorm."),
            mixer=PartSpec("attention", {
                "hidden": h, "n_q_heads": cfg.n_q_heads, "n_kv_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim,
                "position": PartSpec("rope_halves", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta}),
            }, "self_attn."),
            norm2=norm("post_attention_layernorm."),
            ffn=PartSpec("swiglu", {"hidden": h, "intermediate": cfg.intermediate_size}, "mlp."),
        ))
    return ModelPlan(
        hidden_size=h,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("table", {"vocab": cfg.vocab_size, "hidden": h}, "embed_tokens."),
        layers=layers,
        schedule=[LayerCall(i, i) for i in range(cfg.n_layers)],
        final_norm=norm("norm."),
        # a tied head shares the embedding table when the checkpoint stores no lm_head.weight
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": h,
                                 "tied_to": "embed_tokens.weight" if cfg.tie_word_embeddings else None}, "lm_head."),
        ignored_prefixes=("model.vision_model.", "model.connector.", "vision_model.", "connector."),
    )
