"""Configuration reading, refusals, and the architecture registry (CPU)."""

import json

import pytest

from prefixserve_b200.config import (Architecture, LlamaConfig, UnknownArchitectureError, UnsupportedModelError,
                                     architecture_of, get_architecture, read_model_folder, register_architecture,
                                     registered_architectures)
from prefixserve_b200.config.spec import LayerCall, ModelSpec, part

import helpers

BASE = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256, "hidden_size": 2048,
    "intermediate_size": 8192, "num_hidden_layers": 16, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "rms_norm_eps": 1e-5, "max_position_embeddings": 131072, "tie_word_embeddings": True,
    "rope_theta": 500000.0, "eos_token_id": 128001,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
}


def test_reads_every_size_from_the_file():
    cfg = LlamaConfig.from_dicts(BASE)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size, cfg.num_layers) == (128256, 2048, 8192, 16)
    assert (cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.q_size, cfg.kv_size) == (32, 8, 64, 2048, 512)
    assert cfg.rope_theta == 500000.0 and cfg.rope_scaling.factor == 32.0
    assert cfg.rope_scaling.original_max_position_embeddings == 8192
    assert cfg.tie_word_embeddings and cfg.stop_token_ids == frozenset({128001})
    assert cfg.num_parameters == 1235814400


def test_newer_layout_with_rope_parameters():
    raw = {k: v for k, v in BASE.items() if k not in ("rope_theta", "rope_scaling")}
    raw["rope_parameters"] = dict(BASE["rope_scaling"], rope_theta=123456.0)
    cfg = LlamaConfig.from_dicts(raw)
    assert cfg.rope_theta == 123456.0 and cfg.rope_scaling.factor == 32.0


def test_defaults():
    raw = {k: v for k, v in BASE.items() if k not in ("num_key_value_heads", "head_dim", "rope_theta", "rope_scaling",
                                                      "tie_word_embeddings", "eos_token_id")}
    cfg = LlamaConfig.from_dicts(raw)
    assert cfg.num_kv_heads == 32 and cfg.head_dim == 64 and cfg.rope_theta == 10000.0
    assert cfg.rope_scaling is None and not cfg.tie_word_embeddings and cfg.stop_token_ids == frozenset()
    assert LlamaConfig.from_dicts(dict(raw, rope_scaling={"rope_type": "default"})).rope_scaling is None


def test_stop_ids_prefer_generation_config():
    cfg = LlamaConfig.from_dicts(BASE, {"eos_token_id": [128001, 128008, None, 128009]})
    assert cfg.stop_token_ids == frozenset({128001, 128008, 128009})


@pytest.mark.parametrize("change,word", [
    ({"model_type": "mistral"}, "model_type"),
    ({"num_key_value_heads": 5}, "heads"),
    ({"attention_bias": True}, "bias"),
    ({"mlp_bias": True}, "bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "lacks"),
    ({"hidden_size": None}, "lacks"),
])
def test_refusals(change, word):
    with pytest.raises(UnsupportedModelError, match=word):
        LlamaConfig.from_dicts(dict(BASE, **change))


def test_config_json_round_trip(tmp_path):
    for which in helpers.TINY.values():
        cfg = which["cfg"]
        (tmp_path / "config.json").write_text(json.dumps(cfg.to_config_json()))
        arch, back = read_model_folder(tmp_path)
        assert arch.name == "LlamaForCausalLM" and back == cfg


def test_registry_picks_by_architecture_name(tmp_path):
    assert "LlamaForCausalLM" in registered_architectures()
    assert architecture_of({"architectures": ["LlamaForCausalLM"]}).name == "LlamaForCausalLM"
    assert architecture_of({"model_type": "llama"}).name == "LlamaForCausalLM"  # hand-written folders
    with pytest.raises(UnknownArchitectureError, match="registered"):
        architecture_of({"architectures": ["NoSuchModel"]})
    with pytest.raises(UnknownArchitectureError):
        get_architecture("Nope")
    with pytest.raises(FileNotFoundError):
        read_model_folder(tmp_path / "missing")


def test_another_architecture_can_be_registered():
    arch = Architecture("ToyForTests", ("toy",), lambda raw, gen: dict(raw), lambda cfg: None, lambda path: path)
    register_architecture(arch, replace=True)
    assert architecture_of({"architectures": ["ToyForTests"]}) is arch
    with pytest.raises(ValueError, match="already"):
        register_architecture(arch)


def test_llama_spec_is_data():
    arch = get_architecture("LlamaForCausalLM")
    cfg = helpers.TINY_B["cfg"]
    spec = arch.to_spec(cfg)
    assert len(spec.layers) == 3 and [c.layer for c in spec.schedule] == [0, 1, 2]
    mixer = spec.layers[0].mixer
    assert mixer.kind == "attention" and mixer["num_kv_heads"] == 1 and mixer["head_dim"] == 32
    assert mixer["position"].kind == "rope" and mixer["position"]["scaling"]["factor"] == 4.0
    assert spec.layers[0].ffn["intermediate_size"] == 256 and spec.final_norm["eps"] == 1e-6
    assert spec.head["tied"] is False and spec.num_cache_entries == 3
    assert arch.tensor_name("layers.2.mixer.k_proj") == "model.layers.2.self_attn.k_proj.weight"
    assert arch.tensor_name("layers.0.ffn_norm.weight") == "model.layers.0.post_attention_layernorm.weight"


def test_run_list_is_checked():
    arch = get_architecture("LlamaForCausalLM")
    spec = arch.to_spec(helpers.TINY_A["cfg"])
    kw = dict(architecture="x", vocab_size=8, hidden_size=8, max_positions=8, embedding=spec.embedding,
              layers=spec.layers, final_norm=spec.final_norm, head=spec.head)
    ModelSpec(schedule=(LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(1, 0, writes_cache=False)), **kw)
    with pytest.raises(ValueError, match="names layer"):
        ModelSpec(schedule=(LayerCall(5, 0),), **kw)
    with pytest.raises(ValueError, match="before anything wrote"):
        ModelSpec(schedule=(LayerCall(0, 1, writes_cache=False),), **kw)
    with pytest.raises(ValueError, match="written by"):
        ModelSpec(schedule=(LayerCall(0, 0), LayerCall(1, 0)), **kw)
    assert part("rms", size=4, eps=1e-5).with_params(eps=1e-6)["eps"] == 1e-6
