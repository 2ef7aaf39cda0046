"""Replay through the scheduler (prefix hits, preemption and recomputation, steps launched ahead, captured decode
steps), with every sampled token replaced by a given one, against the plain implementation: at the head sizes where
the bfloat16 path runs its tensor-core kernels, in float32 and in bfloat16."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers
import plain_model

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def workload(which: str, seed: int = 0, decode: int = 48):
    """Five requests over one 48-token prefix (three pages), arriving staggered so that later ones find the prefix
    in the cache; each generates ``decode`` given tokens."""
    vocab = helpers.TINY[which]["cfg"].vocab_size
    shared = helpers.random_tokens(vocab, 48, seed=seed + 1)
    arrivals = {0: ["r0"], 4: ["r1", "r2"], 7: ["r3"], 9: ["r4"]}
    requests = {}
    for i, extra in enumerate((70, 9, 101, 33, 140)):
        prompt = shared + helpers.random_tokens(vocab, extra, seed=seed + 10 + i)
        forced = helpers.random_tokens(vocab, decode + 3 * i, seed=seed + 20 + i)
        requests[f"r{i}"] = (prompt, forced)
    return requests, arrivals


def drive(folder, dtype, requests, arrivals, pool_tokens, *, chunk=96, max_running=3, bug=None, **kw):
    """Runs the trace in this process; returns ((request, position) -> logits row, counters, replayer)."""
    from prefixserve_b200.engine.replay import ScheduledReplayer
    rp = ScheduledReplayer(folder, dtype, pool_tokens, chunk=chunk, max_running=max_running, **kw)
    rp.engine.runner.inject_bug = bug
    rows = {}
    step = 0
    left = set(requests)
    while left or step <= max(arrivals):
        record = {"step": step, "add": [{"id": rid, "prompt": requests[rid][0], "forced": requests[rid][1]}
                                        for rid in arrivals.get(step, [])]}
        out, info = rp.run_step(record)
        for k, row in enumerate(info["rows"]):
            rows[(row["id"], row["position"])] = torch.from_numpy(out[k].copy())
        left -= set(info["finished"])
        step += 1
        assert step < 3000, "the trace does not end"
    rp.engine.cache.check()
    return rows, rp.counters(), rp


def judge(cfg, tensors, requests, rows, dtype):
    """Every generated position of every request has a row, and the rows agree with the plain implementation."""
    worst = 0.0
    for rid, (prompt, forced) in requests.items():
        seq = prompt + forced
        want = plain_model.forward(cfg, tensors, seq)[len(prompt) - 1: len(seq) - 1]
        got = torch.stack([rows[(rid, p)] for p in range(len(prompt), len(seq))])
        if dtype == "float32":
            err = float((got - want).abs().max()) / float(want.abs().max())
            worst = max(worst, err / 1e-4)
        else:
            plain_bf16 = plain_model.forward(cfg, tensors, seq, dtype=torch.bfloat16)[len(prompt) - 1: len(seq) - 1]
            ours, theirs = helpers.rel_err(got, want), helpers.rel_err(plain_bf16, want)
            worst = max(worst, ours / 0.15, ours / (1.5 * theirs + 1e-3))
    return worst  # <= 1 passes


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for which in ("D", "E"):
        folder = helpers.make_folder(tmp_path_factory.mktemp(f"tiny{which}16"), which, dtype=torch.bfloat16)
        out[which] = (folder, *plain_model.read_folder(folder))
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["D", "E"])
def test_prefix_hits_steps_ahead_and_captured_steps_match_plain(models, which, dtype, monkeypatch):
    from prefixserve_b200.ops import library, tensorcore
    folder, cfg, tensors = models[which]
    monkeypatch.setattr(tensorcore, "TCGEN05_MIN_TILES", 1)
    monkeypatch.setattr(tensorcore, "TCGEN05_MIN_ROWS", 1)  # tiny matrices: let the tcgen05 product take the portions
    requests, arrivals = workload(which)
    before = library.launch_counts.copy()
    rows, counters, rp = drive(folder, dtype, requests, arrivals, pool_tokens=2048)
    taken = library.launch_counts - before
    assert counters["cached_prompt_tokens"] >= 48 * 3, counters     # r1..r4 found the shared pages
    assert counters["launched_ahead"] > 10 and counters["graph_replays"] > 10 and counters["preemptions"] == 0, counters
    if dtype == "bfloat16":
        for name in ("attention_prefill_tcgen05", "attention_decode", "gemm_tcgen05_rope", "gemm_stream_norm_rope",
                     "gemm_tcgen05_gated", "gemm_stream_norm_gated"):
            assert taken[name] > 0, (name, dict(taken))
        assert library.tcgen05_status() == 0
    assert judge(cfg, tensors, requests, rows, dtype) <= 1.0
    st = rp.scheduler.stats()
    assert st.num_running == 0 and st.free_blocks + st.cached_blocks == rp.engine.num_blocks


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["D", "E"])
def test_preemption_and_recomputation_match_plain(models, which, dtype):
    """A pool one page larger than the longest request needs alone: running requests are preempted, their pages go to
    the prefix tree, and what they computed is found again or recomputed."""
    folder, cfg, tensors = models[which]
    requests, arrivals = workload(which, seed=5, decode=30)
    need = max(-(-(len(p) + len(f)) // 16) for p, f in requests.values())
    rows, counters, _ = drive(folder, dtype, requests, arrivals, pool_tokens=16 * (need + 1), max_running=4)
    assert counters["preemptions"] > 0 and counters["cached_prompt_tokens"] > 0, counters
    assert judge(cfg, tensors, requests, rows, dtype) <= 1.0


@pytest.mark.parametrize("dtype,bug", [("float32", "rope_relative"), ("bfloat16", "rope_relative"), ("bfloat16", "kv_len_short")])
def test_the_comparison_notices_injected_faults(models, dtype, bug):
    """The same judgement must fail when the step function numbers positions from the start of a portion or reports
    one key too few (the faults PrefixServe's suite injects: tests/test_llama_exact.py:227-241).  The float32
    attention kernel masks by position and never reads the key count, so the second fault is a bfloat16 one."""
    folder, cfg, tensors = models["D"]
    requests, arrivals = workload("D")
    rows, _, _ = drive(folder, dtype, requests, arrivals, pool_tokens=2048, bug=bug)
    assert judge(cfg, tensors, requests, rows, dtype) > 1.0, "the injected fault went unnoticed"


def test_scheduler_mode_from_the_command_line(models, tmp_path):
    """bin/trace_run --mode scheduler as a user runs it: stdin lines, done lines, .f32 and .json files, stats line."""
    folder, cfg, tensors = models["D"]
    requests, arrivals = workload("D", decode=20)
    lines = []
    for step in range(90):
        lines.append({"step": step, "add": [{"id": rid, "prompt": requests[rid][0], "forced": requests[rid][1]}
                                            for rid in arrivals.get(step, [])]})
    out = tmp_path / "out"
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--mode", "scheduler", "--model", str(folder), "--dtype", "float32",
           "--out", str(out), "--max-tokens", "2048", "--chunk", "96", "--max-running", "3"]
    proc = subprocess.run(cmd, input="".join(json.dumps(s) + "\n" for s in lines), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    printed = proc.stdout.splitlines()
    assert [ln for ln in printed if ln.startswith("done ")] == [f"done {s['step']}" for s in lines]
    stats = json.loads(next(ln for ln in printed if ln.startswith("stats "))[6:])
    assert stats["cached_prompt_tokens"] > 0 and stats["launched_ahead"] > 0
    vocab = helpers.TINY["D"]["cfg"].vocab_size
    rows = {}
    for s in lines:
        info = json.loads((out / f"{s['step']}.json").read_text())
        if info["rows"]:
            data = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(len(info["rows"]), vocab)
            for k, row in enumerate(info["rows"]):
                rows[(row["id"], row["position"])] = torch.from_numpy(data[k].copy())
    assert judge(cfg, tensors, requests, rows, "float32") <= 1.0
