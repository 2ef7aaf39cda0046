"""A plain, slow Llama: whole sequences, no cache, one function per part.

Written from the formulas of PrefixServe's model code (each function cites
file:line there) and compared once with that code on a tiny random model (see
tests/golden/).  It shares no code with prefixserve_b200: it reads the folder
itself and uses only torch tensor arithmetic on the CPU (or a given device).
Every tensor op runs in ``dtype``; for bfloat16 that reproduces the
reference's rounding after every op.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors.torch import load_file


def read_folder(folder):
    """config.json as a dict, tensors by checkpoint name."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    tensors = load_file(str(folder / "model.safetensors"))
    return cfg, tensors


def sizes(cfg):
    heads = cfg["num_attention_heads"]
    kv_heads = cfg.get("num_key_value_heads", heads)  # prefixserve/model/config.py:67
    head_dim = cfg.get("head_dim") or cfg["hidden_size"] // heads  # prefixserve/model/config.py:72
    return heads, kv_heads, head_dim


def rope_inv_freq(cfg):
    """prefixserve/model/llama.py:24-46 (llama3 scaling: three bands by wavelength)."""
    _, _, dim = sizes(cfg)
    block = cfg.get("rope_parameters") or cfg.get("rope_scaling")  # prefixserve/model/config.py:78
    theta = (cfg.get("rope_parameters") or {}).get("rope_theta", cfg.get("rope_theta"))
    theta = 10000.0 if theta is None else float(theta)  # prefixserve/model/config.py:79-80
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))
    kind = (block or {}).get("rope_type", (block or {}).get("type"))
    if kind in (None, "default"):
        return inv_freq
    assert kind == "llama3", kind
    factor = float(block["factor"])
    low_ff, high_ff = float(block["low_freq_factor"]), float(block["high_freq_factor"])
    old_ctx = block["original_max_position_embeddings"]
    low_freq_wavelen = old_ctx / low_ff
    high_freq_wavelen = old_ctx / high_ff
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_freq_wavelen, inv_freq / factor, inv_freq)
    smooth = (old_ctx / wavelen - low_ff) / (high_ff - low_ff)
    smoothed = (1 - smooth) * scaled / factor + smooth * scaled
    is_medium = ~(wavelen < high_freq_wavelen) * ~(wavelen > low_freq_wavelen)
    return torch.where(is_medium, smoothed, scaled)


def rope_tables(cfg, positions, dtype):
    """cos/sin [len(positions), D] for the given absolute positions; prefixserve/model/llama.py:49-60.

    Computed in float32 and cast at the end.  The reference casts its table to
    the model dtype; ``table_dtype=float32`` is the more exact choice this
    repository's engine makes, so the caller picks which to compare against.
    """
    inv_freq = rope_inv_freq(cfg)
    freqs = torch.outer(positions.to(torch.int64).float(), inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rms_norm(x, weight, eps):
    """prefixserve/model/llama.py:63-69: float32 mean of squares, downcast, then the gain."""
    dtype = x.dtype
    xf = x.to(torch.float32)
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return weight * xf.to(dtype)


def apply_rope(x, cos, sin):
    """x [T, heads, D], cos/sin [T, 1, D]; split-half rotation, prefixserve/model/llama.py:72-77."""
    x1, x2 = x.chunk(2, dim=-1)
    return x * cos + torch.cat((-x2, x1), dim=-1) * sin


def causal_attention(q, k, v, window=None, scale=None):
    """q [T, hq, D], k/v [T, hkv, D] of ONE sequence starting at position 0 -> [T, hq, D].

    prefixserve/model/attention.py:109-120: grouped heads by repeat_interleave,
    scores scaled by 1/sqrt(D) (:75), keys after the query masked with -inf
    (:116-118), softmax in float32 (:119).  ``window`` (not in the reference)
    additionally hides keys more than window-1 positions before the query.
    """
    t, hq, d = q.shape
    group = hq // k.shape[1]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    keys = k.repeat_interleave(group, dim=1)
    vals = v.repeat_interleave(group, dim=1)
    qh = q.transpose(0, 1)  # [H, T, D]
    scores = torch.matmul(qh, keys.permute(1, 2, 0)) * scale  # [H, T, T]
    q_pos = torch.arange(t, device=q.device)[:, None]
    k_pos = torch.arange(t, device=q.device)[None, :]
    hidden = k_pos > q_pos
    if window is not None:
        hidden = hidden | (k_pos <= q_pos - window)
    scores = scores.masked_fill(hidden, float("-inf"))
    probs = torch.softmax(scores, dim=-1, dtype=torch.float32).to(q.dtype)
    return torch.matmul(probs, vals.transpose(0, 1)).transpose(0, 1)


def gated_mlp(x, gate_w, up_w, down_w):
    """prefixserve/model/llama.py:120-121: down(silu(gate(x)) * up(x))."""
    gate = torch.nn.functional.linear(x, gate_w)
    up = torch.nn.functional.linear(x, up_w)
    return torch.nn.functional.linear(torch.nn.functional.silu(gate) * up, down_w)


def attention_block(cfg, x, w, prefix, cos, sin, window=None):
    """prefixserve/model/llama.py:113-117 for one whole sequence."""
    heads, kv_heads, d = sizes(cfg)
    t = x.shape[0]
    q = torch.nn.functional.linear(x, w[prefix + "self_attn.q_proj.weight"]).view(t, heads, d)
    k = torch.nn.functional.linear(x, w[prefix + "self_attn.k_proj.weight"]).view(t, kv_heads, d)
    v = torch.nn.functional.linear(x, w[prefix + "self_attn.v_proj.weight"]).view(t, kv_heads, d)
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    o = causal_attention(q, k, v, window=window)
    return torch.nn.functional.linear(o.reshape(t, heads * d), w[prefix + "self_attn.o_proj.weight"])


def forward(cfg, tensors, token_ids, dtype=torch.float32, device="cpu", rope_table_dtype=None):
    """Logits [T, vocab] (float32) of one whole sequence; prefixserve/model/llama.py:87-126."""
    w = {k: v.to(device=device, dtype=dtype) for k, v in tensors.items()}
    ids = torch.as_tensor(token_ids, dtype=torch.long, device=device)
    t = ids.shape[0]
    eps = cfg["rms_norm_eps"]
    cos, sin = rope_tables(cfg, torch.arange(t), rope_table_dtype or dtype)
    cos, sin = cos.to(device)[:, None, :], sin.to(device)[:, None, :]
    if cos.dtype != dtype:  # float32 tables with bfloat16 activations: rotate in float32, round once
        rot = lambda x: apply_rope(x.float(), cos, sin).to(dtype)  # noqa: E731
    else:
        rot = None
    h = torch.nn.functional.embedding(ids, w["model.embed_tokens.weight"])
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        x = rms_norm(h, w[p + "input_layernorm.weight"], eps)
        if rot is None:
            h = h + attention_block(cfg, x, w, p, cos, sin)
        else:
            h = h + _attention_block_f32_rope(cfg, x, w, p, rot)
        x = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + gated_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    h = rms_norm(h, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return torch.nn.functional.linear(h, head).float()


def _attention_block_f32_rope(cfg, x, w, prefix, rot):
    heads, kv_heads, d = sizes(cfg)
    t = x.shape[0]
    q = rot(torch.nn.functional.linear(x, w[prefix + "self_attn.q_proj.weight"]).view(t, heads, d))
    k = rot(torch.nn.functional.linear(x, w[prefix + "self_attn.k_proj.weight"]).view(t, kv_heads, d))
    v = torch.nn.functional.linear(x, w[prefix + "self_attn.v_proj.weight"]).view(t, kv_heads, d)
    o = causal_attention(q, k, v)
    return torch.nn.functional.linear(o.reshape(t, heads * d), w[prefix + "self_attn.o_proj.weight"])


def greedy(cfg, tensors, prompt, steps, dtype=torch.float32, device="cpu"):
    """Recomputes the whole sequence for every new token (no cache), like the reference's oracle
    (tests/test_llama_exact.py:110-119 of PrefixServe)."""
    seq = list(prompt)
    out = []
    for _ in range(steps):
        logits = forward(cfg, tensors, seq, dtype=dtype, device=device)
        tok = int(torch.argmax(logits[-1]))
        out.append(tok)
        seq.append(tok)
    return out


def gumbel_uniform(seed, position, vocab):
    """The engine's counter-based uniform draw, restated with Python integers."""
    mask = (1 << 64) - 1

    def mix(z):
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        return z ^ (z >> 31)

    a = mix((seed + 0x9E3779B97F4A7C15 * (position + 1)) & mask)
    out = []
    for i in range(vocab):
        r = mix(a ^ ((0xD1B54A32D192ED03 * (i + 1)) & mask))
        out.append(((r >> 40) + 0.5) / 16777216.0)
    return torch.tensor(out, dtype=torch.float32)
