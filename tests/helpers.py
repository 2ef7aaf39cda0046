"""Tiny configurations, model folders and trace builders shared by the tests."""

from __future__ import annotations

import numpy as np
import torch

from prefixserve_b200.config import Llama3RopeScaling, LlamaConfig
from prefixserve_b200.weights import write_random_model

# Two tiny Llamas that differ in every size and option, and a third with awkward sizes.
TINY_A = dict(
    cfg=LlamaConfig(vocab_size=256, hidden_size=64, intermediate_size=128, num_layers=2, num_heads=4, num_kv_heads=2,
                    head_dim=16, rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None, max_position_embeddings=256,
                    tie_word_embeddings=True),
    seed=0, std=0.02, gain_noise=0.0)
TINY_B = dict(
    cfg=LlamaConfig(vocab_size=384, hidden_size=96, intermediate_size=256, num_layers=3, num_heads=3, num_kv_heads=1,
                    head_dim=32, rms_norm_eps=1e-6, rope_theta=500000.0,
                    rope_scaling=Llama3RopeScaling(4.0, 1.0, 4.0, 64), max_position_embeddings=512,
                    tie_word_embeddings=False),
    seed=1, std=0.02, gain_noise=0.1)
TINY_C = dict(
    cfg=LlamaConfig(vocab_size=333, hidden_size=80, intermediate_size=112, num_layers=1, num_heads=5, num_kv_heads=5,
                    head_dim=48, rms_norm_eps=3e-5, rope_theta=777.0,
                    rope_scaling=Llama3RopeScaling(8.0, 1.0, 2.0, 16), max_position_embeddings=300,
                    tie_word_embeddings=False),
    seed=2, std=0.2, gain_noise=0.2)
# head size 64: the size at which the bfloat16 path runs the tensor-core attention kernels
TINY_D = dict(
    cfg=LlamaConfig(vocab_size=300, hidden_size=128, intermediate_size=160, num_layers=2, num_heads=4, num_kv_heads=2,
                    head_dim=64, rms_norm_eps=1e-5, rope_theta=50000.0,
                    rope_scaling=Llama3RopeScaling(2.0, 1.0, 4.0, 32), max_position_embeddings=1024,
                    tie_word_embeddings=True),
    seed=3, std=0.08, gain_noise=0.1)
# head size 128, one key/value head for three query heads: the other size the tensor-core attention kernels are built for
TINY_E = dict(
    cfg=LlamaConfig(vocab_size=411, hidden_size=192, intermediate_size=224, num_layers=2, num_heads=3, num_kv_heads=1,
                    head_dim=128, rms_norm_eps=2e-6, rope_theta=123456.0,
                    rope_scaling=Llama3RopeScaling(16.0, 1.0, 8.0, 48), max_position_embeddings=2048,
                    tie_word_embeddings=False),
    seed=4, std=0.06, gain_noise=0.15)
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}


def make_folder(tmp, which: str, dtype=torch.float32):
    spec = TINY[which]
    return write_random_model(tmp, spec["cfg"], spec["seed"], std=spec["std"], gain_noise=spec["gain_noise"], dtype=dtype)


def random_tokens(vocab: int, n: int, seed: int) -> list[int]:
    return [int(t) for t in np.random.RandomState(seed).randint(0, vocab, size=n)]


# ---- traces ------------------------------------------------------------------

def trace_whole(seqs: dict[str, list[int]]):
    """Each request alone and whole: one step, every position wanted."""
    steps = []
    for i, (rid, toks) in enumerate(seqs.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def trace_tail_decode(seqs: dict[str, list[int]], tail: int = 32):
    """Most of it in one step, the last ``tail`` tokens one by one."""
    steps = []
    n = 0
    for rid, toks in seqs.items():
        head = max(len(toks) - tail, 1)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        n += 1
        for p in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
            n += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(seqs: dict[str, list[int]], sizes=(7, 2, 16, 3, 2, 5, 17, 2, 31, 4)):
    """Portions of changing size, down to two tokens."""
    steps = []
    n = 0
    for rid, toks in seqs.items():
        at = k = 0
        while at < len(toks):
            size = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[at:at + size], "want": list(range(size))}],
                          "end": [rid] if at + size == len(toks) else []})
            at += size
            n += 1
    return steps


def trace_mixed(seqs: dict[str, list[int]], max_live: int = 4, seed: int = 0, prefill_to: float = 0.6):
    """Up to ``max_live`` requests at once: portions of some beside single tokens of others.

    A request first gets portions of random size until ``prefill_to`` of its
    length, then one token per step; a finished request makes room for the next,
    so with a small pool its pages are used again.  Requests sit out a step now and then.
    """
    rng = np.random.RandomState(seed)
    waiting = list(seqs.items())
    live: list[list] = []  # [rid, toks, at]
    steps = []
    n = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live.append([rid, toks, 0])
        entries, ended = [], []
        for rec in live:
            rid, toks, at = rec
            if len(live) > 1 and rng.rand() < 0.15:
                continue  # left out of this step, goes on later
            if at < int(prefill_to * len(toks)):
                size = int(rng.choice([2, 3, 5, 8, 16, 19, 33]))
                size = max(1, min(size, int(prefill_to * len(toks)) - at))
            else:
                size = 1
            size = min(size, len(toks) - at)
            entries.append({"id": rid, "tokens": toks[at:at + size], "want": list(range(size))})
            rec[2] = at + size
            if rec[2] == len(toks):
                ended.append(rid)
        live = [rec for rec in live if rec[2] < len(rec[1])]
        steps.append({"step": n, "entries": entries, "end": ended})
        n += 1
    return steps


def trace_many_live(seqs: dict[str, list[int]], tail: int = 12, portion_beside: bool = True):
    """Every request live at once: request k's prompt (all but its last ``tail`` tokens) arrives in step k in one
    portion beside single decoded tokens of the requests before it; then all decode together until they end, the
    shorter ones first.  With dozens of requests the decode steps have dozens of rows."""
    order = list(seqs.items())
    at = {rid: 0 for rid, _ in order}
    steps = []
    n = 0
    started = 0
    while any(at[rid] < len(toks) for rid, toks in order):
        entries, ended = [], []
        for k, (rid, toks) in enumerate(order):
            if k < started and at[rid] < len(toks):
                entries.append({"id": rid, "tokens": [toks[at[rid]]], "want": [0]})
                at[rid] += 1
            elif k == started:
                head = max(len(toks) - tail, 1)
                entries.append({"id": rid, "tokens": toks[:head], "want": [head - 1] if portion_beside else list(range(head))})
                at[rid] = head
            else:
                continue
            if at[rid] == len(toks):
                ended.append(rid)
        started = min(started + 1, len(order))
        steps.append({"step": n, "entries": entries, "end": ended})
        n += 1
    return steps


def peak_tokens(steps, page: int = 64) -> int:
    """Most tokens live requests hold at any time, each rounded up to a multiple of ``page``."""
    held: dict[str, int] = {}
    peak = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-v // page) * page for v in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def collect(steps, outputs):
    """outputs: step number -> array [wanted, vocab].  Returns (request id, position) -> logits row."""
    pos: dict[str, int] = {}
    rows = {}
    for st in steps:
        out = outputs.get(st["step"])
        k = 0
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                rows[(e["id"], base + w)] = out[k]
                k += 1
            pos[e["id"]] = base + len(e["tokens"])
        for rid in st["end"]:
            pos.pop(rid, None)
        assert out is None or k == out.shape[0]
    return rows


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """Mean over rows of |g - w| / |w| (the reference's bfloat16 acceptance measure,
    tests/gpu/test_engine_flashinfer.py:86-108 of PrefixServe)."""
    got, want = got.double(), want.double()
    return float(((got - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-12)).mean())
