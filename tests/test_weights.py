"""Weights by tensor name: placement rules, the one error that lists everything, random-weights mode (CPU)."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from prefixserve_b200.config import read_model_folder
from prefixserve_b200.parts import build_model
from prefixserve_b200.weights import WeightLoadError, held_dtype, load_tensors, write_random_model

import helpers


def load(folder, dtype=torch.bfloat16):
    arch, cfg = read_model_folder(folder)
    model = build_model(arch.to_spec(cfg))
    return load_tensors(folder, model.param_table(), arch.tensor_name, lambda n: arch.ignorable(cfg, n),
                        compute_dtype=dtype, device="cpu"), model


def test_random_mode_writes_a_loadable_folder(tmp_path):
    folder = helpers.make_folder(tmp_path, "B", dtype=torch.bfloat16)
    assert sorted(p.name for p in folder.iterdir()) == ["config.json", "model.safetensors"]
    raw = load_file(str(folder / "model.safetensors"))
    assert "lm_head.weight" in raw and raw["model.layers.2.mlp.down_proj.weight"].shape == (96, 256)
    assert all(t.dtype == torch.bfloat16 for t in raw.values())
    tensors, model = load(folder)
    assert tensors["layers.0.mixer.q_proj"].dtype == torch.bfloat16
    assert tensors["layers.0.mixer_norm.weight"].dtype == torch.float32  # gains are widened (exact)
    assert set(tensors) == set(model.param_table())


def test_random_mode_is_deterministic(tmp_path):
    a = load_file(str(helpers.make_folder(tmp_path / "a", "A") / "model.safetensors"))
    b = load_file(str(helpers.make_folder(tmp_path / "b", "A") / "model.safetensors"))
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    assert "lm_head.weight" not in a  # tied
    assert torch.equal(a["model.norm.weight"], torch.ones(64))
    c = load_file(str(helpers.make_folder(tmp_path / "c", "B") / "model.safetensors"))
    assert not torch.equal(c["model.norm.weight"], torch.ones(96))  # gains 1 + noise
    assert abs(float(a["model.embed_tokens.weight"].std()) - 0.02) < 2e-3


def test_placement_rules():
    bf, f32 = torch.bfloat16, torch.float32
    assert held_dtype("matrix", bf, bf) == bf
    assert held_dtype("matrix", torch.float16, bf) == bf
    assert held_dtype("matrix", f32, bf) == f32          # stored in 32-bit: stays so
    assert held_dtype("vector", bf, bf) == f32
    assert held_dtype("matrix", bf, f32) == f32          # the 32-bit path widens everything
    assert held_dtype("table_int", torch.int64, bf) == torch.int32
    assert held_dtype("matrix", torch.int64, bf) == torch.int32


def test_float32_checkpoint_stays_float32_on_the_bfloat16_path(tmp_path):
    folder = helpers.make_folder(tmp_path, "A", dtype=torch.float32)
    tensors, _ = load(folder, torch.bfloat16)
    assert tensors["embedding.weight"].dtype == torch.float32
    tensors32, _ = load(folder, torch.float32)
    assert all(t.dtype == torch.float32 for t in tensors32.values())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = helpers.make_folder(tmp_path, "B")
    path = folder / "model.safetensors"
    raw = load_file(str(path))
    del raw["model.layers.1.self_attn.k_proj.weight"]
    del raw["model.norm.weight"]
    raw["model.layers.0.mlp.up_proj.weight"] = torch.zeros(255, 96)
    raw["model.layers.0.self_attn.qkv_proj.weight"] = torch.zeros(2, 2)
    raw["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)  # harmless, rebuilt from the config
    save_file(raw, str(path))
    with pytest.raises(WeightLoadError) as err:
        load(folder)
    msg = str(err.value)
    assert "missing (2)" in msg and "model.layers.1.self_attn.k_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected (1)" in msg and "qkv_proj" in msg and "inv_freq" not in msg
    assert "wrong shape (1)" in msg and "(255, 96)" in msg and "(256, 96)" in msg


def test_tied_model_may_carry_a_head_copy(tmp_path):
    folder = helpers.make_folder(tmp_path, "A")
    path = folder / "model.safetensors"
    raw = load_file(str(path))
    raw["lm_head.weight"] = raw["model.embed_tokens.weight"].clone()
    save_file(raw, str(path))
    load(folder)  # no error


def test_untied_model_needs_its_head(tmp_path):
    folder = helpers.make_folder(tmp_path, "B")
    path = folder / "model.safetensors"
    raw = load_file(str(path))
    del raw["lm_head.weight"]
    save_file(raw, str(path))
    with pytest.raises(WeightLoadError, match="lm_head.weight"):
        load(folder)


def test_sharded_checkpoint(tmp_path):
    folder = helpers.make_folder(tmp_path, "A")
    raw = load_file(str(folder / "model.safetensors"))
    names = sorted(raw)
    half = len(names) // 2
    save_file({k: raw[k] for k in names[:half]}, str(folder / "part-1.safetensors"))
    save_file({k: raw[k] for k in names[half:]}, str(folder / "part-2.safetensors"))
    (folder / "model.safetensors").unlink()
    index = {"weight_map": {k: ("part-1.safetensors" if i < half else "part-2.safetensors") for i, k in enumerate(names)}}
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    tensors, model = load(folder)
    assert set(tensors) == set(model.param_table())


def test_no_weights_at_all(tmp_path):
    folder = helpers.make_folder(tmp_path, "A")
    (folder / "model.safetensors").unlink()
    with pytest.raises(WeightLoadError, match="neither"):
        load(folder)


def test_float32_checkpoint_can_be_rounded_at_load_as_the_reference_does(tmp_path):
    """prefixserve/model/weights.py:94-98 casts every tensor to the engine's type; here that is an option."""
    folder = helpers.make_folder(tmp_path, "A", dtype=torch.float32)
    arch, cfg = read_model_folder(folder)
    model = build_model(arch.to_spec(cfg))
    tensors = load_tensors(folder, model.param_table(), arch.tensor_name, lambda n: arch.ignorable(cfg, n),
                           compute_dtype=torch.bfloat16, device="cpu", cast_float32=True)
    assert tensors["embedding.weight"].dtype == torch.bfloat16
    assert tensors["layers.0.mixer.q_proj"].dtype == torch.bfloat16
    assert tensors["layers.0.mixer_norm.weight"].dtype == torch.float32   # gains stay wide either way
    assert held_dtype("matrix", torch.float32, torch.bfloat16, cast_float32=True) == torch.bfloat16
    assert held_dtype("matrix", torch.float32, torch.float32, cast_float32=True) == torch.float32


@pytest.mark.parametrize("which,tied", [("A", True), ("B", False)])
def test_weight_bytes_count_a_tied_head_once(tmp_path, which, tied):
    """prefixserve/model/weights.py:49-59: the footprint of the loaded weights, shared tensors once."""
    folder = helpers.make_folder(tmp_path, which, dtype=torch.bfloat16)
    tensors, model = load(folder)
    model.load(tensors, compute_dtype=torch.bfloat16, device=torch.device("cpu"), max_positions=64)
    cfg = helpers.TINY[which]["cfg"]
    q, kv = cfg.num_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
    matrices = cfg.vocab_size * cfg.hidden_size * (1 if tied else 2) + cfg.num_layers * (
        (q + 2 * kv) * cfg.hidden_size + cfg.hidden_size * q + 3 * cfg.hidden_size * cfg.intermediate_size)
    gains = (2 * cfg.num_layers + 1) * cfg.hidden_size
    assert model.num_bytes() == 2 * matrices + 4 * gains   # bfloat16 matrices, float32 gains
    assert (model.head.weight.data_ptr() == model.embedding.table.data_ptr()) == tied
