"""Weights: the safetensors container, the loader's one clear error, the random-weights mode (CPU)."""

from __future__ import annotations

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

import plain_llama as plain
from edgerag_b200.config import DecoderConfig
from edgerag_b200.models.decoder import DecoderModel
from edgerag_b200.models.llama import llama_plan
from edgerag_b200.weights.loader import WeightsError, load_safetensors, random_tensors, write_model_folder
from edgerag_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

CPU = torch.device("cpu")


def _model(raw):
    cfg = DecoderConfig.from_dict(raw)
    return cfg, DecoderModel(llama_plan(cfg), torch.float32, CPU)


def test_container_round_trip_against_the_library(tmp_path):
    tensors = {"a.w": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
               "t": torch.arange(6, dtype=torch.int32).view(2, 3), "h": torch.randn(2, 2).half()}
    write_safetensors(tmp_path / "x.safetensors", tensors, {"k": "v"})
    theirs = load_file(str(tmp_path / "x.safetensors"))
    for k, v in tensors.items():
        assert torch.equal(theirs[k], v) and theirs[k].dtype == v.dtype
    save_file(tensors, str(tmp_path / "y.safetensors"))
    with SafetensorsFile(tmp_path / "y.safetensors") as f:
        assert sorted(f.names()) == sorted(tensors)
        for k, v in tensors.items():
            assert f.shape(k) == tuple(v.shape) and f.dtype(k) == v.dtype and torch.equal(f.tensor(k).clone(), v)
    (tmp_path / "bad.safetensors").write_bytes(b"\xff" * 4)
    with pytest.raises(SafetensorsError):
        SafetensorsFile(tmp_path / "bad.safetensors")


def test_loader_reads_by_name_and_keeps_types(tmp_path):
    folder = plain.write_model_folder(tmp_path / "a", plain.TINY_A, 0)
    cfg, model = _model(plain.TINY_A)
    got = load_safetensors(folder, model.weight_specs(), torch.bfloat16, CPU)
    theirs = load_file(str(folder / "model.safetensors"))
    assert got["layers.1.mlp.up_proj.weight"].dtype == torch.bfloat16
    assert torch.equal(got["layers.1.mlp.up_proj.weight"], theirs["model.layers.1.mlp.up_proj.weight"].bfloat16())
    # norm weights are held in float32 (the stored values, exactly); a tied head shares the table
    assert got["norm.weight"].dtype == torch.float32 and torch.equal(got["norm.weight"], theirs["model.norm.weight"])
    assert got["lm_head.weight"] is got["embed_tokens.weight"]
    model.load_weights(load_safetensors(folder, model.weight_specs(), torch.float32, CPU))
    assert model.head.weight.data_ptr() == model.embedding.weight.data_ptr()
    assert model.blocks[0].mixer.w_qkv.shape == ((4 + 2 * 2) * 16, 64)


def test_one_error_lists_every_offender(tmp_path):
    folder = plain.write_model_folder(tmp_path / "b", plain.TINY_B, 1)
    tensors = {k: v.clone() for k, v in load_file(str(folder / "model.safetensors")).items()}
    del tensors["model.layers.2.mlp.down_proj.weight"], tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(32, 95)
    tensors["model.layers.9.extra.weight"] = torch.zeros(2)
    tensors["model.vision_model.patch.weight"] = torch.zeros(2)   # another tower: not an error
    save_file(tensors, str(folder / "model.safetensors"))
    cfg, model = _model(plain.TINY_B)
    plan = llama_plan(cfg)
    with pytest.raises(WeightsError) as info:
        load_safetensors(folder, model.weight_specs(), torch.float32, CPU, plan.name_prefixes, plan.ignored_prefixes)
    err = info.value
    assert err.missing == ["layers.2.mlp.down_proj.weight", "lm_head.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 95), (32, 96))]
    text = str(err)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "[32, 95]", "expected [32, 96]"):
        assert needle in text


def test_prefixes_of_composite_checkpoints(tmp_path):
    folder = plain.write_model_folder(tmp_path / "b", plain.TINY_B, 1)
    tensors = {k: v.clone() for k, v in load_file(str(folder / "model.safetensors")).items()}
    renamed = {k.replace("model.", "model.text_model.", 1) if k.startswith("model.") else k: v for k, v in tensors.items()}
    save_file(renamed, str(folder / "model.safetensors"))
    cfg, model = _model(plain.TINY_B)
    got = load_safetensors(folder, model.weight_specs(), torch.float32, CPU)
    assert torch.equal(got["embed_tokens.weight"], tensors["model.embed_tokens.weight"])


def test_sharded_checkpoints_load_through_their_index(tmp_path):
    """A folder with model.safetensors.index.json and shards gives the same tensors as the single file;
    a shard the index names but the folder lacks, and a tensor missing from every shard, are reported."""
    folder = plain.write_model_folder(tmp_path / "b", plain.TINY_B, 1)
    tensors = {k: v.clone() for k, v in load_file(str(folder / "model.safetensors")).items()}
    cfg, model = _model(plain.TINY_B)
    whole = load_safetensors(folder, model.weight_specs(), torch.float32, CPU)
    names = sorted(tensors)
    shards = {"model-00001-of-00003.safetensors": names[0::3], "model-00002-of-00003.safetensors": names[1::3],
              "model-00003-of-00003.safetensors": names[2::3]}
    (folder / "model.safetensors").unlink()
    for shard, members in shards.items():
        save_file({n: tensors[n] for n in members}, str(folder / shard))
    index = {"metadata": {"total_size": 0}, "weight_map": {n: shard for shard, members in shards.items() for n in members}}
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    got = load_safetensors(folder, model.weight_specs(), torch.float32, CPU)
    assert sorted(got) == sorted(whole) and all(torch.equal(got[n], whole[n]) for n in whole)

    # a tensor that no shard holds: the one error, with its name
    lost = "model.layers.1.mlp.up_proj.weight"
    shard = index["weight_map"].pop(lost)
    save_file({n: tensors[n] for n in shards[shard] if n != lost}, str(folder / shard))
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(WeightsError) as info:
        load_safetensors(folder, model.weight_specs(), torch.float32, CPU)
    assert info.value.missing == ["layers.1.mlp.up_proj.weight"]
    # a shard file that is not there
    (folder / "model-00002-of-00003.safetensors").unlink()
    with pytest.raises(WeightsError, match="model-00002-of-00003.safetensors"):
        load_safetensors(folder, model.weight_specs(), torch.float32, CPU)
    # neither a single file nor an index
    with pytest.raises(SafetensorsError, match="does not exist"):
        load_safetensors(tmp_path / "nowhere", model.weight_specs(), torch.float32, CPU)


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    cfg, model = _model(plain.TINY_A)
    folder = write_model_folder(tmp_path / "r", cfg.to_hf_dict(), model.weight_specs(), seed=3, dtype=torch.bfloat16)
    assert json.loads((folder / "config.json").read_text())["num_hidden_layers"] == 2
    stored = load_file(str(folder / "model.safetensors"))
    assert "lm_head.weight" not in stored and stored["model.embed_tokens.weight"].dtype == torch.bfloat16
    got = load_safetensors(folder, model.weight_specs(), torch.bfloat16, CPU)
    again = random_tensors(model.weight_specs(), 3, compute_dtype=torch.bfloat16)
    other = random_tensors(model.weight_specs(), 4, compute_dtype=torch.bfloat16)
    for name in ("embed_tokens.weight", "layers.1.self_attn.o_proj.weight"):
        assert torch.equal(got[name], again[name]) and not torch.equal(got[name], other[name])
    assert float(got["layers.0.mlp.gate_proj.weight"].float().std()) == pytest.approx(0.02, rel=0.1)
    assert torch.equal(got["norm.weight"], torch.ones(64))
    # the plain implementation reads the same folder
    logits = plain.forward(plain.read_weights(folder), plain.read_config(folder), [1, 2, 3])
    assert logits.shape == (3, 512) and torch.isfinite(logits).all()
