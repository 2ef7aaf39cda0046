"""LlamaForCausalLM as a list of parts.

Dense decoder, pre-norm blocks: RMSNorm -> grouped-query attention with
rotary positions (optionally llama3-scaled) -> residual; RMSNorm -> SiLU-gated
feed-forward -> residual; final RMSNorm; LM head tied to the embedding or not
(prefixserve/model/llama.py:107-126).  Checkpoint names are those the
reference reads (prefixserve/model/weights.py:111-136).
"""

from __future__ import annotations

import re

from ..config.llama import LlamaConfig
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, part, sequential_schedule


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    scaling = None
    if cfg.rope_scaling is not None:
        s = cfg.rope_scaling
        scaling = {
            "kind": "llama3",
            "factor": s.factor,
            "low_freq_factor": s.low_freq_factor,
            "high_freq_factor": s.high_freq_factor,
            "original_max_positions": s.original_max_position_embeddings,
        }
    position = part("rope", head_dim=cfg.head_dim, theta=cfg.rope_theta, scaling=scaling, layout="half")
    norm = part("rms", size=cfg.hidden_size, eps=cfg.rms_norm_eps)
    layer = LayerSpec(
        mixer=part(
            "attention",
            hidden_size=cfg.hidden_size,
            num_heads=cfg.num_heads,
            num_kv_heads=cfg.num_kv_heads,
            head_dim=cfg.head_dim,
            position=position,
            window=None,
        ),
        ffn=part("gated_mlp", hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size, activation="silu"),
        mixer_norm=norm,
        ffn_norm=norm,
        arrangement="pre_norm",
    )
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_positions=cfg.max_position_embeddings,
        embedding=part("token_embedding", vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size),
        layers=(layer,) * cfg.num_layers,
        schedule=sequential_schedule(cfg.num_layers),
        final_norm=norm,
        head=part("lm_head", vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, tied=cfg.tie_word_embeddings),
        stop_token_ids=cfg.stop_token_ids,
    )


_LAYER = re.compile(r"^layers\.(\d+)\.(.+)$")
_IN_LAYER = {
    "mixer_norm.weight": "input_layernorm.weight",
    "ffn_norm.weight": "post_attention_layernorm.weight",
    "mixer.q_proj": "self_attn.q_proj.weight",
    "mixer.k_proj": "self_attn.k_proj.weight",
    "mixer.v_proj": "self_attn.v_proj.weight",
    "mixer.o_proj": "self_attn.o_proj.weight",
    "ffn.gate_proj": "mlp.gate_proj.weight",
    "ffn.up_proj": "mlp.up_proj.weight",
    "ffn.down_proj": "mlp.down_proj.weight",
}
_TOP = {
    "embedding.weight": "model.embed_tokens.weight",
    "final_norm.weight": "model.norm.weight",
    "head.weight": "lm_head.weight",
}


def llama_tensor_name(path: str) -> str:
    if path in _TOP:
        return _TOP[path]
    m = _LAYER.match(path)
    if m and m.group(2) in _IN_LAYER:
        return f"model.layers.{m.group(1)}.{_IN_LAYER[m.group(2)]}"
    raise KeyError(f"LlamaForCausalLM has no tensor for part path {path!r}")


def llama_ignorable(cfg: LlamaConfig, name: str) -> bool:
    # Rotary buffers are rebuilt from the config; a tied model may still
    # carry a copy of its head (prefixserve/model/weights.py:137-141).
    if name.endswith("rotary_emb.inv_freq"):
        return True
    return cfg.tie_word_embeddings and name == "lm_head.weight"


LLAMA = Architecture(
    name="LlamaForCausalLM",
    model_types=("llama",),
    read_config=LlamaConfig.from_dicts,
    to_spec=llama_spec,
    tensor_name=llama_tensor_name,
    ignorable=llama_ignorable,
)

register_architecture(LLAMA, replace=True)
