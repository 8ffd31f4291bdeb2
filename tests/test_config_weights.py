"""Configuration contract, registry, strict weight loading and the random-weights mode (CPU)."""

from __future__ import annotations

import json
import math

import pytest
import torch
from safetensors.torch import load_file, save_file

import helpers

import miniserve_b200  # noqa: F401
from miniserve_b200.config import (Qwen3Config, UnsupportedModelError, load_model_config, register_architecture,
                                   registered_architectures, resolve_architecture)
from miniserve_b200.parts import DecoderModel
from miniserve_b200.weights import WeightLoadError, load_tensors, random_tensors, write_random_model


def test_config_reads_every_size_and_never_infers_head_dim():
    config = Qwen3Config.from_dict(dict(helpers.TINY_B, hidden_size=1024, num_attention_heads=16, head_dim=128))
    assert config.head_dim == 128 and config.hidden_size // config.num_attention_heads == 64
    assert Qwen3Config.from_dict(config.to_dict()) == config
    with pytest.raises(ValueError, match="head_dim"):
        Qwen3Config.from_dict({k: v for k, v in helpers.TINY_A.items() if k != "head_dim"})


@pytest.mark.parametrize("key,value", [
    ("attention_bias", True), ("mlp_bias", True), ("attention_dropout", 0.1), ("hidden_act", "gelu"),
    ("rope_scaling", {"type": "linear", "factor": 2.0}), ("rope_interleaved", True), ("use_sliding_window", True),
    ("hidden_size", 64.0), ("hidden_size", True), ("vocab_size", 0), ("num_key_value_heads", 3), ("head_dim", 15), ("head_dim", 514),
    ("rms_norm_eps", float("nan")), ("rms_norm_eps", 0.0), ("rope_theta", -1.0), ("rope_theta", "1e6"),
    ("tie_word_embeddings", "yes")])
def test_config_rejections(key, value):
    with pytest.raises(ValueError):
        Qwen3Config.from_dict(dict(helpers.TINY_A, **{key: value}))


def test_registry_names_known_architectures():
    assert "Qwen3ForCausalLM" in registered_architectures()
    for bad in ({"architectures": ["LlamaForCausalLM"], "model_type": "llama"}, {"architectures": []},
                {"architectures": ["Qwen3ForCausalLM", "X"]}, {}):
        with pytest.raises(UnsupportedModelError, match="Qwen3ForCausalLM"):
            resolve_architecture(bad)
    with pytest.raises(UnsupportedModelError):
        Qwen3Config.from_dict(dict(helpers.TINY_A, model_type="qwen2"))


def test_registry_accepts_a_new_architecture(tmp_path):
    from miniserve_b200.architectures.qwen3 import build_qwen3_spec

    class ToyConfig(Qwen3Config):
        @classmethod
        def from_dict(cls, data):
            return Qwen3Config.from_dict(dict(data, architectures=["Qwen3ForCausalLM"], model_type="qwen3"))

    register_architecture("ToyForCausalLM", ToyConfig, build_qwen3_spec)
    folder = tmp_path / "toy"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(dict(helpers.TINY_A, architectures=["ToyForCausalLM"])))
    architecture, config = load_model_config(folder)
    assert architecture.name == "ToyForCausalLM" and config.hidden_size == 64


def model_for(name, dtype=torch.bfloat16):
    architecture = resolve_architecture(helpers.TINY[name])
    config = architecture.config_class.from_dict(helpers.TINY[name])
    spec = architecture.build_spec(config)
    return spec, DecoderModel(spec, dtype, "cpu")


def test_random_folder_is_seeded_and_loads(tmp_path):
    a = write_random_model(tmp_path / "m1", helpers.TINY_B, seed=5)
    b = write_random_model(tmp_path / "m2", helpers.TINY_B, seed=5)
    c = write_random_model(tmp_path / "m3", helpers.TINY_B, seed=6)
    ta, tb, tc = (load_file(str(p / "model.safetensors")) for p in (a, b, c))
    assert all(torch.equal(ta[k], tb[k]) for k in ta) and any(not torch.equal(ta[k], tc[k]) for k in ta)
    assert all(t.dtype == torch.bfloat16 for t in ta.values())
    spec, model = model_for("b")
    tensors, report = load_tensors(a, model.param_specs(), torch.bfloat16, "cpu", spec.optional_names)
    assert report.loaded_tensors == len(ta) == 3 + 11 * 3 and "lm_head.weight" in tensors
    norm = ta["model.layers.0.self_attn.q_norm.weight"].float()
    assert 0.05 < float(norm.std()) < 0.2 and abs(float(norm.mean()) - 1) < 0.1
    assert abs(float(ta["model.embed_tokens.weight"].float().std()) - 0.02) < 0.005
    model.load(tensors)
    assert model.blocks[0].mixer.qkv_weight.shape == ((6 + 2 * 2) * 32, 96)
    assert json.loads((a / "config.json").read_text())["head_dim"] == 32


def test_kept_types(tmp_path):
    """bfloat16 stays bfloat16; a vector stored in 32 bits stays float32; float32 compute widens exactly."""
    folder = write_random_model(tmp_path / "m", helpers.TINY_A, seed=1)
    stored = {k: v.clone() for k, v in load_file(str(folder / "model.safetensors")).items()}
    stored["model.norm.weight"] = stored["model.norm.weight"].float() + 1e-4
    save_file(stored, str(folder / "model.safetensors"))
    spec, model = model_for("a")
    tensors, report = load_tensors(folder, model.param_specs(), torch.bfloat16, "cpu", spec.optional_names)
    assert tensors["model.norm.weight"].dtype == torch.float32 and report.kept_float32 == ["model.norm.weight"]
    assert torch.equal(tensors["model.norm.weight"], stored["model.norm.weight"])
    assert tensors["model.layers.0.input_layernorm.weight"].dtype == torch.bfloat16
    assert tensors["model.embed_tokens.weight"].dtype == torch.bfloat16
    wide, _ = load_tensors(folder, model.param_specs(), torch.float32, "cpu", spec.optional_names)
    assert all(t.dtype == torch.float32 for t in wide.values())
    assert torch.equal(wide["model.embed_tokens.weight"], stored["model.embed_tokens.weight"].float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_random_model(tmp_path / "m", helpers.TINY_B, seed=1)
    stored = {k: v.clone() for k, v in load_file(str(folder / "model.safetensors")).items()}
    del stored["model.layers.1.mlp.up_proj.weight"], stored["lm_head.weight"]
    stored["model.layers.7.mlp.up_proj.weight"] = torch.zeros(2, 2)
    stored["extra.bias"] = torch.zeros(3)
    stored["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(16, dtype=torch.bfloat16)
    stored["model.embed_tokens.weight"] = torch.zeros(384, 95, dtype=torch.bfloat16)
    save_file(stored, str(folder / "model.safetensors"))
    spec, model = model_for("b")
    with pytest.raises(WeightLoadError) as caught:
        load_tensors(folder, model.param_specs(), torch.bfloat16, "cpu", spec.optional_names)
    error = caught.value
    assert error.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert error.unexpected == ["extra.bias", "model.layers.7.mlp.up_proj.weight"]
    assert len(error.wrong_shapes) == 2 and "model.embed_tokens.weight: stored (384, 95), model (384, 96)" in error.wrong_shapes
    for text in ("missing tensors (2)", "unexpected tensors (2)", "wrong shapes (2)", "q_norm"):
        assert text in str(error)


def test_tied_output_matrix(tmp_path):
    folder = write_random_model(tmp_path / "m", helpers.TINY_A, seed=1)
    stored = {k: v.clone() for k, v in load_file(str(folder / "model.safetensors")).items()}
    assert "lm_head.weight" not in stored
    spec, model = model_for("a")
    tied = [("lm_head.weight", spec.embedding_name)]
    stored["lm_head.weight"] = stored["model.embed_tokens.weight"].clone()     # stored copy of the tied matrix: accepted
    save_file(stored, str(folder / "model.safetensors"))
    tensors, _ = load_tensors(folder, model.param_specs(), torch.bfloat16, "cpu", spec.optional_names, tied)
    model.load(tensors)
    assert model.output_weight is model.embedding
    stored["lm_head.weight"][3, 3] += 1                                        # ... unless it differs
    save_file(stored, str(folder / "model.safetensors"))
    with pytest.raises(WeightLoadError, match="tied"):
        load_tensors(folder, model.param_specs(), torch.bfloat16, "cpu", spec.optional_names, tied)


def test_sharded_folder_and_duplicates(tmp_path):
    folder = write_random_model(tmp_path / "m", helpers.TINY_A, seed=1)
    stored = {k: v.clone() for k, v in load_file(str(folder / "model.safetensors")).items()}
    names = sorted(stored)
    (folder / "model.safetensors").unlink()
    save_file({k: stored[k] for k in names[:5]}, str(folder / "model-00001-of-00002.safetensors"))
    save_file({k: stored[k] for k in names[5:]}, str(folder / "model-00002-of-00002.safetensors"))
    weight_map = {k: "model-00001-of-00002.safetensors" for k in names[:5]}
    weight_map.update({k: "model-00002-of-00002.safetensors" for k in names[5:]})
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    spec, model = model_for("a")
    tensors, _ = load_tensors(folder, model.param_specs(), torch.bfloat16, "cpu", spec.optional_names)
    assert sorted(tensors) == names
    save_file({k: stored[k] for k in names[4:]}, str(folder / "model-00002-of-00002.safetensors"))
    with pytest.raises(WeightLoadError, match="appears in"):
        load_tensors(folder, model.param_specs(), torch.bfloat16, "cpu", spec.optional_names)
    (folder / "model-00002-of-00002.safetensors").unlink()
    with pytest.raises(FileNotFoundError):
        load_tensors(folder, model.param_specs(), torch.bfloat16, "cpu", spec.optional_names)


def test_kernel_choices_can_be_kept_in_a_file(tmp_path, monkeypatch):
    """MINISERVE_B200_CHOICES_FILE: what was measured once is written down and used by later runs instead of a new
    measurement, so that the order of a product's sums (and with it bfloat16 results) repeats; entries that name
    no known kernel are ignored."""
    import json

    from miniserve_b200 import kernels

    path = tmp_path / "choices.json"
    monkeypatch.setattr(kernels, "CHOICES_FILE", str(path))
    assert kernels._stored_choice("linear", 4096, 2048) is None
    kernels._store_choice("linear", 4096, 2048, "wide")
    kernels._store_choice("gated", 12288, 2048, "separate")
    assert kernels._stored_choice("linear", 4096, 2048) == "wide" and kernels._stored_choice("gated", 12288, 2048) == "separate"
    assert json.loads(path.read_text()) == {"linear 4096x2048": "wide", "gated 12288x2048": "separate"}
    path.write_text('{"linear 8x8": "no such kernel"}')
    assert kernels._stored_choice("linear", 8, 8) is None
    path.write_text("not json")
    assert kernels._stored_choice("linear", 8, 8) is None
    kernels._store_choice("linear", 8, 8, "skinny")
    assert kernels._stored_choice("linear", 8, 8) == "skinny"
