"""What bench.py promises before it touches a GPU: its answers to runs it does not do, and the record it writes."""

import importlib.util
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def _bench(*args, env=None):
    full = dict(os.environ)
    for key in ("WORLD_SIZE", "RANK", "LOCAL_RANK"):
        full.pop(key, None)
    full.update(env or {})
    done = subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, env=full, cwd=ROOT)
    lines = [ln for ln in done.stdout.splitlines() if ln.strip()]
    return done.returncode, lines


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_more_than_one_gpu_is_one_line_and_exit_code_two():
    code, lines = _bench("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert code == 2 and len(lines) == 1
    said = json.loads(lines[0])
    assert said["n_gpus"] == 2 and "one GPU" in said["unsupported"]


def test_under_a_launcher_only_the_first_rank_speaks():
    code, lines = _bench("--gpus", "2", env={"WORLD_SIZE": "2", "RANK": "1", "LOCAL_RANK": "1"})
    assert code == 2 and lines == []
    code, lines = _bench("--gpus", "2", env={"WORLD_SIZE": "2", "RANK": "0", "LOCAL_RANK": "0"})
    assert code == 2 and len(lines) == 1
    # a world of two is refused even if the flag says one
    code, lines = _bench(env={"WORLD_SIZE": "2", "RANK": "0"})
    assert code == 2 and len(lines) == 1


def test_options_that_do_not_go_together_are_refused():
    for args in (("--only", "prefill", "--prompt", "9000"),                 # longer than the context
                 ("--prompt", "1024"),                                       # not with the whole bench
                 ("--model", "8b"),                                          # the headline stays at its sizes
                 ("--profile",)):                                            # needs --only
        code, lines = _bench(*args)
        assert code == 2 and len(lines) == 1 and "unsupported" in json.loads(lines[0]), args


@pytest.mark.skipif(torch.cuda.is_available(), reason="a machine without a GPU is what this is about")
def test_without_a_gpu_each_arm_says_so_in_one_line():
    code, lines = _bench("--steps", "2")
    assert code == 1 and len(lines) == 1 and "no CUDA device" in json.loads(lines[0])["error"]
    code, lines = _bench("--impl", "reference", "--steps", "2")
    said = json.loads(lines[0])
    assert code == 0 and len(lines) == 1 and said["impl"] == "reference" and "unavailable" in said


def test_the_config_record_is_flat_short_and_names_every_size(bench):
    block = bench.config_block(bench.FULL_LAYERS, 8)
    assert len(block) <= 20
    assert all(isinstance(v, (int, float, str, bool)) for v in block.values()), "deeper values are lost in the record"
    model = bench.MODEL
    assert block["layers"] == block["layers_full"] == bench.FULL_LAYERS == model["num_hidden_layers"]
    assert (block["hidden"], block["intermediate"], block["vocab"]) == (model["hidden_size"], model["intermediate_size"], model["vocab_size"])
    assert (block["heads"], block["kv_heads"], block["head_dim"]) == (model["num_attention_heads"], model["num_key_value_heads"], model["head_dim"])
    assert block["global_batch"] == 8 and block["seq_len"] == bench.CONTEXT and block["prefill_tokens"] == bench.PREFILL_TOKENS
    fewer = bench.config_block(4, 8)
    assert fewer["layers"] == 4 and fewer["layers_full"] == bench.FULL_LAYERS, "fewer layers must show beside the full count"


def test_flops_and_bytes_of_a_step_by_hand(bench):
    m = bench.MODEL
    h, i, v = m["hidden_size"], m["intermediate_size"], m["vocab_size"]
    q, kv = m["num_attention_heads"] * m["head_dim"], m["num_key_value_heads"] * m["head_dim"]
    layers, t, prefix = 3, 512, 1536
    products = 2 * t * layers * (h * (q + 2 * kv) + q * h + 3 * h * i) + 2 * h * v   # the last row's logits only
    # every new token attends to the prefix and, causally, to (t + 1) / 2 of the new ones on average: Q K^T and P V
    attention = layers * 4 * t * (prefix + (t + 1) / 2) * q
    assert bench.prefill_flops(t, layers, prefix) == pytest.approx(products + attention, rel=1e-12)
    assert bench.prefill_flops(t, layers) < bench.prefill_flops(t, layers, prefix)
    # keys and values of one token in every layer, bfloat16
    assert bench.kv_bytes_per_token(layers) == layers * 2 * kv * 2
