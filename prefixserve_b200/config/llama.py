"""Typed Llama configuration, read from the keys of a model folder's config.json.

Same keys, defaults and refusals as the reference's reader
(prefixserve/model/config.py:54-120): ``model_type`` must be ``llama``;
``num_key_value_heads`` defaults to the number of query heads and must divide
it; ``head_dim`` defaults to ``hidden_size // num_attention_heads``; the rope
base and scaling are read either from the top level (``rope_theta``,
``rope_scaling``) or from one ``rope_parameters`` dictionary; only the
``llama3`` scaling (or none) is understood; biases are refused; stop ids come
from ``generation_config.json`` first.  Every size used anywhere in the engine
comes from here.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping


class UnsupportedModelError(ValueError):
    """The folder describes something this engine cannot run."""


@dataclass(frozen=True)
class Llama3RopeScaling:
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


_REQUIRED = (
    "vocab_size",
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
    "rms_norm_eps",
    "max_position_embeddings",
)


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Llama3RopeScaling | None
    max_position_embeddings: int
    tie_word_embeddings: bool
    stop_token_ids: frozenset[int] = frozenset()

    architecture = "LlamaForCausalLM"

    def __post_init__(self) -> None:
        bad = []
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_layers", "num_heads",
                     "num_kv_heads", "head_dim", "max_position_embeddings"):
            if int(getattr(self, name)) < 1:
                bad.append(f"{name}={getattr(self, name)} must be positive")
        if not bad and self.num_heads % self.num_kv_heads:
            bad.append(f"{self.num_heads} query heads cannot be shared among {self.num_kv_heads} key/value heads")
        if not bad and self.head_dim % 2:
            bad.append(f"head_dim {self.head_dim} must be even for rotary pairs")
        if not self.rms_norm_eps > 0:
            bad.append(f"rms_norm_eps={self.rms_norm_eps} must be positive")
        if bad:
            raise UnsupportedModelError("; ".join(bad))

    # ---- derived sizes -------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def num_parameters(self) -> int:
        h, i = self.hidden_size, self.intermediate_size
        per_layer = 2 * h + (self.q_size + 2 * self.kv_size) * h + h * self.q_size + 3 * h * i
        head = 0 if self.tie_word_embeddings else self.vocab_size * h
        return self.vocab_size * h + self.num_layers * per_layer + h + head

    # ---- reading -------------------------------------------------------
    @classmethod
    def from_dir(cls, folder: str | Path) -> "LlamaConfig":
        folder = Path(folder)
        raw = json.loads((folder / "config.json").read_text())
        gen_file = folder / "generation_config.json"
        gen = json.loads(gen_file.read_text()) if gen_file.exists() else None
        return cls.from_dicts(raw, gen)

    @classmethod
    def from_dicts(cls, raw: Mapping[str, Any], gen: Mapping[str, Any] | None = None) -> "LlamaConfig":
        if raw.get("model_type") != "llama":
            raise UnsupportedModelError(f"model_type {raw.get('model_type')!r} is not 'llama'")
        absent = [k for k in _REQUIRED if raw.get(k) is None]
        if absent:
            raise UnsupportedModelError(f"config.json lacks {', '.join(absent)}")
        if raw.get("attention_bias") or raw.get("mlp_bias"):
            raise UnsupportedModelError("attention_bias / mlp_bias are set; projections with biases are not built")

        heads = int(raw["num_attention_heads"])
        hidden = int(raw["hidden_size"])
        kv_heads = raw.get("num_key_value_heads")
        head_dim = raw.get("head_dim")

        # The rope base and its scaling live either at the top level or, in
        # newer files, together in one "rope_parameters" dictionary.
        rope_block = raw.get("rope_parameters")
        scaling_raw = rope_block if rope_block else raw.get("rope_scaling")
        theta = (rope_block or {}).get("rope_theta", raw.get("rope_theta"))

        eos = raw.get("eos_token_id")
        if gen is not None and "eos_token_id" in gen:
            eos = gen["eos_token_id"]
        if not isinstance(eos, (list, tuple)):
            eos = [eos]

        return cls(
            vocab_size=int(raw["vocab_size"]),
            hidden_size=hidden,
            intermediate_size=int(raw["intermediate_size"]),
            num_layers=int(raw["num_hidden_layers"]),
            num_heads=heads,
            num_kv_heads=int(kv_heads) if kv_heads is not None else heads,
            head_dim=int(head_dim) if head_dim else hidden // heads,
            rms_norm_eps=float(raw["rms_norm_eps"]),
            rope_theta=float(theta) if theta is not None else 10000.0,
            rope_scaling=_read_scaling(scaling_raw),
            max_position_embeddings=int(raw["max_position_embeddings"]),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            stop_token_ids=frozenset(int(t) for t in eos if t is not None),
        )

    # ---- writing (random-weights mode) ----------------------------------
    def to_config_json(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_layers,
            "num_attention_heads": self.num_heads,
            "num_key_value_heads": self.num_kv_heads,
            "head_dim": self.head_dim,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.rope_scaling is not None:
            s = self.rope_scaling
            out["rope_scaling"] = {
                "rope_type": "llama3",
                "factor": s.factor,
                "low_freq_factor": s.low_freq_factor,
                "high_freq_factor": s.high_freq_factor,
                "original_max_position_embeddings": s.original_max_position_embeddings,
            }
        stops = sorted(self.stop_token_ids)
        if stops:
            out["eos_token_id"] = stops[0] if len(stops) == 1 else stops
        return out


def _read_scaling(block: Mapping[str, Any] | None) -> Llama3RopeScaling | None:
    if not block:
        return None
    kind = block.get("rope_type", block.get("type"))
    if kind in (None, "default"):
        return None
    if kind != "llama3":
        raise UnsupportedModelError(f"rope scaling of type {kind!r} is not built (only 'llama3' or none)")
    wanted = ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")
    absent = [k for k in wanted if k not in block]
    if absent:
        raise UnsupportedModelError(f"llama3 rope scaling lacks {', '.join(absent)}")
    return Llama3RopeScaling(
        factor=float(block["factor"]),
        low_freq_factor=float(block["low_freq_factor"]),
        high_freq_factor=float(block["high_freq_factor"]),
        original_max_position_embeddings=int(block["original_max_position_embeddings"]),
    )
