"""The plain implementation itself: against the stored output of PrefixServe's own model code, and its parts (CPU)."""

import json
import math
from pathlib import Path

import pytest
import torch

import plain_model
import tiny_model

GOLDEN = Path(__file__).resolve().parent / "golden" / "tiny_llama_reference_logits.json"


def test_matches_the_reference_model_code(tmp_path):
    gold = json.loads(GOLDEN.read_text())
    tiny_model.write(tmp_path)
    cfg, tensors = plain_model.read_folder(tmp_path)
    got = plain_model.forward(cfg, tensors, gold["tokens"])
    want = torch.tensor(gold["logits"]).view(*gold["shape"])
    assert float((got - want).abs().max()) <= 1e-5 * float(want.abs().max())
    assert gold["max_abs_whole_vs_portions"] < 1e-5  # the reference's own paged path agreed with its whole-prompt path


def test_rope_bands():
    cfg = dict(tiny_model.CONFIG, head_dim=32)
    cfg["rope_scaling"] = dict(cfg["rope_scaling"], original_max_position_embeddings=64)
    plain = dict(cfg, rope_scaling=None)
    ratio = plain_model.rope_inv_freq(cfg) / plain_model.rope_inv_freq(plain)
    assert ratio[0] == 1 and abs(float(ratio[-1]) - 0.25) < 1e-6  # short waves kept, long ones divided by the factor
    assert ((ratio > 0.25 + 1e-6) & (ratio < 1 - 1e-6)).any()     # and a blended band between


def test_rms_norm_and_rotation_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    out = plain_model.rms_norm(x, torch.tensor([2.0, 0.5]), 0.0)
    assert torch.allclose(out, torch.tensor([[2 * 3 / math.sqrt(12.5), 0.5 * 4 / math.sqrt(12.5)]]))
    v = torch.tensor([[[1.0, 0.0]]])  # one head, D=2: a rotation by the angle
    ang = torch.tensor(0.3)
    r = plain_model.apply_rope(v, ang.cos().view(1, 1, 1).expand(1, 1, 2), ang.sin().view(1, 1, 1).expand(1, 1, 2))
    assert torch.allclose(r, torch.tensor([[[math.cos(0.3), math.sin(0.3)]]]))


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    out = plain_model.causal_attention(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])  # first token sees only itself
    changed = v.clone()
    changed[5] += 1
    assert torch.allclose(plain_model.causal_attention(q, k, changed)[:5], out[:5])  # no look-ahead
    w1 = plain_model.causal_attention(q, k, v, window=1)
    assert torch.allclose(w1, v.repeat_interleave(2, dim=1))  # a window of one is the token's own value


def test_greedy_generation_recomputes(tmp_path):
    tiny_model.write(tmp_path)
    cfg, tensors = plain_model.read_folder(tmp_path)
    toks = plain_model.greedy(cfg, tensors, [1, 2, 3], 4)
    again = plain_model.forward(cfg, tensors, [1, 2, 3] + toks[:3])
    assert toks[3] == int(again[-1].argmax())


def test_gumbel_draws_are_uniform():
    u = plain_model.gumbel_uniform(5, 9, 4000)
    assert 0 < float(u.min()) and float(u.max()) < 1 and abs(float(u.mean()) - 0.5) < 0.02
    assert not torch.equal(u, plain_model.gumbel_uniform(5, 10, 4000))
