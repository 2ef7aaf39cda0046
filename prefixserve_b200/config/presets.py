"""Named configurations for the random-weights mode (benchmarks and tests).

These are config.json contents, i.e. data: the engine reads sizes only from a
configuration, never from this file directly.
"""

from __future__ import annotations

from .llama import LlamaConfig

_LLAMA3_ROPE = {"rope_type": "llama3", "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                "original_max_position_embeddings": 8192}

PRESETS: dict[str, dict] = {
    "tiny-a": {
        "model_type": "llama", "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
        "max_position_embeddings": 256, "tie_word_embeddings": True,
    },
    "tiny-b": {
        "model_type": "llama", "vocab_size": 384, "hidden_size": 96, "intermediate_size": 256, "num_hidden_layers": 3,
        "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32, "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 64},
        "max_position_embeddings": 512, "tie_word_embeddings": False,
    },
    "llama-3.2-1b": {
        "model_type": "llama", "vocab_size": 128256, "hidden_size": 2048, "intermediate_size": 8192,
        "num_hidden_layers": 16, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
        "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "rope_scaling": dict(_LLAMA3_ROPE, factor=32.0),
        "max_position_embeddings": 131072, "tie_word_embeddings": True,
    },
    "llama-3.2-3b": {
        "model_type": "llama", "vocab_size": 128256, "hidden_size": 3072, "intermediate_size": 8192,
        "num_hidden_layers": 28, "num_attention_heads": 24, "num_key_value_heads": 8, "head_dim": 128,
        "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "rope_scaling": dict(_LLAMA3_ROPE, factor=32.0),
        "max_position_embeddings": 131072, "tie_word_embeddings": True,
    },
    "llama-3.1-8b": {
        "model_type": "llama", "vocab_size": 128256, "hidden_size": 4096, "intermediate_size": 14336,
        "num_hidden_layers": 32, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
        "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "rope_scaling": dict(_LLAMA3_ROPE, factor=8.0),
        "max_position_embeddings": 131072, "tie_word_embeddings": False,
    },
}


def preset(name: str) -> LlamaConfig:
    try:
        return LlamaConfig.from_dicts(PRESETS[name])
    except KeyError:
        raise ValueError(f"no preset {name!r}; known: {sorted(PRESETS)}") from None
