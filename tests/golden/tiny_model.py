"""Deterministic tiny Llama folders for anchoring the plain implementation (test-only)."""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch
from safetensors.torch import save_file

CONFIG = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 160,
    "hidden_size": 48,
    "intermediate_size": 80,
    "num_hidden_layers": 2,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 32},
    "max_position_embeddings": 256,
    "tie_word_embeddings": False,
}
SEED = 7
TOKENS = [int(t) for t in np.random.RandomState(11).randint(0, 160, size=45)]


def tensor_shapes(cfg):
    h, i = cfg["hidden_size"], cfg["intermediate_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    shapes = {"model.embed_tokens.weight": (cfg["vocab_size"], h)}
    for n in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{n}."
        shapes[p + "input_layernorm.weight"] = (h,)
        shapes[p + "self_attn.q_proj.weight"] = (q, h)
        shapes[p + "self_attn.k_proj.weight"] = (kv, h)
        shapes[p + "self_attn.v_proj.weight"] = (kv, h)
        shapes[p + "self_attn.o_proj.weight"] = (h, q)
        shapes[p + "post_attention_layernorm.weight"] = (h,)
        shapes[p + "mlp.gate_proj.weight"] = (i, h)
        shapes[p + "mlp.up_proj.weight"] = (i, h)
        shapes[p + "mlp.down_proj.weight"] = (h, i)
    shapes["model.norm.weight"] = (h,)
    if not cfg.get("tie_word_embeddings", False):
        shapes["lm_head.weight"] = (cfg["vocab_size"], h)
    return shapes


def write(folder, cfg=CONFIG, seed=SEED, std=0.15):
    """Writes config.json + model.safetensors (float32); matrices N(0, std), gains 1 + N(0, 0.1)."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    rng = np.random.RandomState(seed)
    tensors = {}
    for name, shape in tensor_shapes(cfg).items():
        if len(shape) == 1:
            arr = 1.0 + 0.1 * rng.standard_normal(shape)
        else:
            arr = std * rng.standard_normal(shape)
        tensors[name] = torch.from_numpy(arr.astype(np.float32))
    save_file(tensors, str(folder / "model.safetensors"), metadata={"format": "pt"})
    (folder / "config.json").write_text(json.dumps(cfg, indent=2))
    return folder
