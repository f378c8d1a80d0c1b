"""Configuration and registry (CPU)."""

from __future__ import annotations

import copy
import json

import pytest

import plain_llama as plain
from edgerag_b200.config import (ConfigError, DecoderConfig, architecture_names, architecture_of,
                                 read_model_folder, register_architecture)


def test_flat_and_composite_configs():
    a = DecoderConfig.from_dict(plain.TINY_A)
    assert (a.n_layers, a.hidden_size, a.n_q_heads, a.n_kv_heads, a.head_dim) == (2, 64, 4, 2, 16)
    assert a.tie_word_embeddings and a.rope_theta == 10000.0 and a.rms_norm_eps == 1e-5 and a.n_rep == 2
    b = DecoderConfig.from_dict(plain.TINY_B)
    assert (b.n_layers, b.hidden_size, b.n_q_heads, b.n_kv_heads, b.head_dim) == (3, 96, 3, 1, 32)
    assert not b.tie_word_embeddings and b.rope_theta == 100000.0 and b.rms_norm_eps == 1e-6
    assert b.pad_token_id == 2 and b.vocab_size == 1000 and b.intermediate_size == 256


def test_defaults_follow_the_reference():
    raw = copy.deepcopy(plain.TINY_A)
    del raw["num_key_value_heads"], raw["head_dim"]
    c = DecoderConfig.from_dict(raw)
    assert c.n_kv_heads == c.n_q_heads == 4 and c.head_dim == 16   # edgerag/core/spec.py:209-219


def test_kv_bytes_match_the_reference_figures():
    """edgerag tests/test_spec.py: 196,608 and 23,040 bytes per token in 16-bit."""
    big = DecoderConfig("LlamaForCausalLM", 24, 2048, 32, 32, 64, 8192, 49155, 273768.0, 1e-5, 8192, True)
    small = DecoderConfig("LlamaForCausalLM", 30, 576, 9, 3, 64, 1536, 49280, 1e5, 1e-5, 8192, True)
    assert big.kv_bytes_per_token(2) == 196608 and small.kv_bytes_per_token(2) == 23040


@pytest.mark.parametrize("mutate, needle", [
    (lambda r: r.pop("rope_theta"), "rope_theta"),
    (lambda r: r.pop("hidden_size"), "hidden_size"),
    (lambda r: r.update(num_key_value_heads=3), "divisible"),
    (lambda r: r.update(pad_token_id=512), "pad_token_id"),
    (lambda r: r.update(hidden_act="gelu"), "activation"),
    (lambda r: r.update(head_dim=15), "odd"),
    (lambda r: r.update(vocab_size=0), "positive"),
    # options that change the arithmetic and are not built: refused by the key's name, never ignored
    (lambda r: r.update(rope_scaling={"rope_type": "llama3", "factor": 8.0}), "rope_scaling"),
    (lambda r: r.update(rope_scaling={"type": "linear", "factor": 2.0}), "rope_scaling"),
    (lambda r: (r.pop("rope_theta"), r.update(rope_parameters={"rope_theta": 1e4, "rope_type": "yarn"})), "rope_type"),
    (lambda r: (r.pop("rope_theta"), r.update(rope_parameters={"rope_theta": 1e4, "partial_rotary_factor": 0.5})), "partial_rotary"),
    (lambda r: r.update(partial_rotary_factor=0.25), "partial_rotary"),
    (lambda r: r.update(attention_bias=True), "attention_bias"),
    (lambda r: r.update(mlp_bias=True), "mlp_bias"),
    (lambda r: r.update(sliding_window=4096), "sliding_window"),
    (lambda r: r.update(use_sliding_window=True, sliding_window=128), "sliding_window"),
    (lambda r: r.update(final_logit_softcapping=30.0), "softcapping"),
])
def test_bad_configs_are_refused(mutate, needle):
    raw = copy.deepcopy(plain.TINY_A)
    mutate(raw)
    with pytest.raises(ConfigError, match=needle):
        DecoderConfig.from_dict(raw)


def test_neutral_values_of_unbuilt_options_are_accepted():
    """What a stock Llama or SmolVLM config.json writes when the option is off must still load."""
    raw = copy.deepcopy(plain.TINY_A)
    raw.update(rope_scaling=None, attention_bias=False, mlp_bias=False, sliding_window=None, use_sliding_window=False)
    assert DecoderConfig.from_dict(raw) == DecoderConfig.from_dict(plain.TINY_A)
    raw.pop("rope_theta")
    raw["rope_parameters"] = {"rope_theta": 10000.0, "rope_type": "default"}
    assert DecoderConfig.from_dict(raw) == DecoderConfig.from_dict(plain.TINY_A)
    raw.update(sliding_window=4096, use_sliding_window=False)      # a window that the config itself switches off
    assert DecoderConfig.from_dict(raw) == DecoderConfig.from_dict(plain.TINY_A)


def test_round_trip_and_folder(tmp_path):
    c = DecoderConfig.from_dict(plain.TINY_B)
    assert DecoderConfig.from_dict(c.to_hf_dict()) == DecoderConfig.from_dict(
        {**c.to_hf_dict(), "architectures": ["SmolVLMForConditionalGeneration"]})
    (tmp_path / "config.json").write_text(json.dumps(plain.TINY_A))
    arch, cfg = read_model_folder(tmp_path)
    assert arch.name == "LlamaForCausalLM" and cfg == DecoderConfig.from_dict(plain.TINY_A)
    assert DecoderConfig.from_json(tmp_path) == cfg
    with pytest.raises(ConfigError):
        read_model_folder(tmp_path / "nowhere")


def test_registry():
    assert {"LlamaForCausalLM", "SmolVLMForConditionalGeneration"} <= set(architecture_names())
    assert architecture_of({"model_type": "smolvlm"}).name == "smolvlm"
    with pytest.raises(ConfigError, match="no registered architecture"):
        architecture_of({"architectures": ["NopeForCausalLM"]})
    register_architecture("NopeForCausalLM", lambda raw, where: raw, lambda cfg: cfg)
    assert architecture_of({"architectures": ["NopeForCausalLM"]}).make_plan(5) == 5


def test_plan_names_every_size_from_the_config():
    from edgerag_b200.models.llama import llama_plan

    cfg = DecoderConfig.from_dict(plain.TINY_B)
    plan = llama_plan(cfg)
    assert len(plan.layers) == 3 and [c.layer for c in plan.schedule] == [0, 1, 2]
    mixer = plan.layers[1].mixer
    assert mixer.kind == "attention" and mixer.params["n_kv_heads"] == 1 and mixer.params["head_dim"] == 32
    assert mixer.params["position"].params == {"head_dim": 32, "theta": 100000.0}
    assert plan.layers[0].norm1.params == {"size": 96, "eps": 1e-6}
    assert plan.head.params["tied_to"] is None
