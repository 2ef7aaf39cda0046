"""Runs PrefixServe's own model code on a tiny random Llama (CPU, float32) and
stores its logits, so that tests/plain_model.py can be checked against the
reference itself rather than against formulas alone.

Needs the reference installed under baseline/_ref (pip install --no-deps
--target baseline/_ref <copy of the reference>).  Run from the repo root:

    python tests/golden/make_golden.py

Writes tests/golden/tiny_llama_reference_logits.json (a few tens of KB): the
logits of every position of one 45-token sequence computed in a single
whole-prompt step, and the logits of its last token when the same sequence is
fed in portions of 16 through the reference's scheduler-free engine path
(paged cache, TorchRefAttention).
"""

import json
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
sys.path.insert(0, str(Path(__file__).resolve().parent))

import tiny_model  # noqa: E402
from prefixserve.model.attention import AttnMetadata, TorchRefAttention  # noqa: E402
from prefixserve.model.config import LlamaConfig  # noqa: E402
from prefixserve.model.llama import LlamaModel  # noqa: E402
from prefixserve.model.weights import load_llama_weights  # noqa: E402


def run(folder, tokens, portions):
    cfg = LlamaConfig.from_dir(folder)
    dev = torch.device("cpu")
    weights = load_llama_weights(folder, cfg, dev, torch.float32)
    model = LlamaModel(cfg, weights, 256, dev, torch.float32)
    attn = TorchRefAttention(cfg.num_heads, cfg.num_kv_heads, cfg.head_dim)
    kv = torch.zeros((cfg.num_layers, 8, 2, 16, cfg.num_kv_heads, cfg.head_dim))
    table = [5, 2, 7, 0, 3]  # pages deliberately out of order
    rows = []
    start = 0
    for n in portions:
        end = start + n
        pages = -(-end // 16)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32)  # noqa: E731
        meta = AttnMetadata(n, 1, i32([0, n]), i32([0, pages]), i32(table[:pages]), i32([end - (pages - 1) * 16]),
                            i32([0, n]), i32([0, pages]), i32(table[:pages]), i32([end - (pages - 1) * 16]))
        attn.plan(meta)
        logits = model.forward(i32(tokens[start:end]), torch.arange(start, end, dtype=torch.int32), kv, attn,
                               torch.arange(n, dtype=torch.int32))
        rows.append(logits)
        start = end
    return torch.cat(rows)


def main():
    with tempfile.TemporaryDirectory() as d:
        tiny_model.write(d)
        tokens = tiny_model.TOKENS
        whole = run(d, tokens, [len(tokens)])
        cut = run(d, tokens, [16, 16, 13])
    assert torch.allclose(whole, cut, atol=1e-5), (whole - cut).abs().max()
    out = {
        "made_by": "tests/golden/make_golden.py with PrefixServe's LlamaModel + TorchRefAttention, CPU float32",
        "seed": tiny_model.SEED,
        "tokens": tokens,
        "shape": list(whole.shape),
        "logits": [round(float(x), 7) for x in whole.flatten().tolist()],
        "max_abs_whole_vs_portions": float((whole - cut).abs().max()),
    }
    path = Path(__file__).resolve().parent / "tiny_llama_reference_logits.json"
    path.write_text(json.dumps(out))
    print(path, path.stat().st_size, "bytes; max |logit|", float(whole.abs().max()))


if __name__ == "__main__":
    main()
