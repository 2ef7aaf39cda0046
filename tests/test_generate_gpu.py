"""Generation through the Python entry point, the scheduler and the command line (GPU)."""

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


@pytest.fixture(scope="module")
def sharp(tmp_path_factory):
    """Tiny B with large weights: clear arg max, so token-exact comparison is meaningful."""
    from prefixserve_b200.weights import write_random_model
    folder = tmp_path_factory.mktemp("sharpB")
    write_random_model(folder, helpers.TINY_B["cfg"], seed=11, std=0.2, gain_noise=0.1, dtype=torch.float32)
    return folder, plain_model.read_folder(folder)


def prompts_b():
    vocab = helpers.TINY_B["cfg"].vocab_size
    shared = helpers.random_tokens(vocab, 32, seed=1)
    return [shared[:1], shared[:16], shared + helpers.random_tokens(vocab, 8, 2), shared + helpers.random_tokens(vocab, 38, 3)]


def test_greedy_generation_matches_plain_in_float32(sharp):
    from prefixserve_b200 import LLM, SamplingParams
    folder, (cfg, tensors) = sharp
    prompts = prompts_b()
    llm = LLM(folder, dtype="float32", max_seq_len=256, num_blocks=24, max_running_requests=3, chunked_prefill_size=24)
    got = llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    want = [plain_model.greedy(cfg, tensors, p, 12) for p in prompts]
    assert got == want
    llm.engine.cache.check()
    st = llm.stats()
    assert st.num_running == 0 and st.free_blocks + st.cached_blocks == 24
    # the same prompts again: now the shared prefix is found in the cache, tokens unchanged
    again = llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    assert again == want and llm.stats().cached_prompt_tokens > 0


def test_preemption_and_recompute_keep_the_tokens(sharp):
    from prefixserve_b200 import LLM, SamplingParams
    folder, (cfg, tensors) = sharp
    vocab = helpers.TINY_B["cfg"].vocab_size
    prompts = [helpers.random_tokens(vocab, n, seed=40 + n) for n in (50, 45, 40)]
    need = -(-(50 + 30) // 16)
    llm = LLM(folder, dtype="float32", max_seq_len=256, num_blocks=need + 3, max_running_requests=3, chunked_prefill_size=32)
    got = llm.generate(prompts, SamplingParams(max_tokens=30, ignore_eos=True))
    assert llm.stats().preemptions > 0
    assert got == [plain_model.greedy(cfg, tensors, p, 30) for p in prompts]
    llm.engine.cache.check()


def test_bfloat16_generation_teacher_forced(sharp):
    """bfloat16 logits along the float32 path's own tokens stay close to float32 truth (the reference's criterion,
    tests/gpu/test_engine_flashinfer.py:86-108 of PrefixServe)."""
    from prefixserve_b200.engine import Engine, EngineConfig, Scheduler
    folder, (cfg, tensors) = sharp
    prompts = prompts_b()
    truth_tokens = [plain_model.greedy(cfg, tensors, p, 10) for p in prompts]
    engine = Engine(EngineConfig(model_path=folder, dtype=torch.bfloat16, max_num_seqs=4, max_prefill_tokens=24,
                                 max_seq_len=256, num_blocks=32))
    engine.capture_logits = True
    sched = Scheduler(engine.cache, chunk_size=24)
    for i, p in enumerate(prompts):
        sched.add_request(f"r{i}", p, 10, ignore_eos=True)
    rows = {f"r{i}": [] for i in range(len(prompts))}
    while sched.has_work():
        batch = sched.schedule_step(24, 4)
        engine.step(batch)
        forced = {}
        for w in batch.work:
            if w.samples:
                rid = w.req.req_id
                rows[rid].append(engine.last_logits[rid])
                forced[rid] = truth_tokens[int(rid[1:])][len(w.req.output)]
        sched.commit(batch, forced)
    for i, p in enumerate(prompts):
        seq = p + truth_tokens[i]
        want = plain_model.forward(cfg, tensors, seq)[len(p) - 1: len(seq) - 1]
        plain_bf16 = plain_model.forward(cfg, tensors, seq, dtype=torch.bfloat16)[len(p) - 1: len(seq) - 1]
        got = torch.stack(rows[f"r{i}"])
        ours, theirs = helpers.rel_err(got, want), helpers.rel_err(plain_bf16, want)
        assert ours < 0.15 and ours <= 1.5 * theirs + 1e-3, (i, ours, theirs)


def test_stop_ids_and_cached_pages_are_never_written(sharp):
    from prefixserve_b200.engine import Engine, EngineConfig, Scheduler
    folder, (cfg, tensors) = sharp
    prompt = helpers.random_tokens(helpers.TINY_B["cfg"].vocab_size, 20, seed=9)
    first = plain_model.greedy(cfg, tensors, prompt, 3)
    engine = Engine(EngineConfig(model_path=folder, dtype=torch.float32, max_num_seqs=2, max_prefill_tokens=16,
                                 max_seq_len=128, num_blocks=16))
    sched = Scheduler(engine.cache, chunk_size=16, stop_token_ids=[first[2]])
    sched.add_request("a", prompt, 10)
    out = []
    while sched.has_work():
        batch = sched.schedule_step(16, 2)
        for w in batch.work:  # a step never writes a position whose page the prefix cache owns
            table = sched.block_table(w.req)
            for pos in range(w.start, w.end):
                assert not engine.cache.is_cached(table[pos // 16])
        res = sched.commit(batch, engine.step(batch))
        out += list(res.new_tokens.values())
    assert out == first[: first.index(first[2]) + 1]  # the stop token is kept, nothing after it


def test_steps_launched_ahead_give_the_same_tokens(sharp):
    """The entry point launches a decode step before it has read the tokens of the one before; a loop that waits for
    every step must produce the same, with greedy and with seeded sampling, and when a stop token ends a request
    one step before the host finds out."""
    from prefixserve_b200 import LLM, SamplingParams
    from prefixserve_b200.engine import Engine, EngineConfig, Scheduler
    folder, (cfg, tensors) = sharp
    vocab = helpers.TINY_B["cfg"].vocab_size
    prompts = [helpers.random_tokens(vocab, n, seed=70 + n) for n in (5, 33, 18)]
    want = [plain_model.greedy(cfg, tensors, p, 20) for p in prompts]
    stop = want[1][7]                                        # ends request 1 early (and whoever else meets it)
    for dtype in ("float32", "bfloat16"):
        for params in (SamplingParams(max_tokens=20), SamplingParams(max_tokens=20, temperature=0.8, seed=5)):
            engine = Engine(EngineConfig(model_path=folder, dtype=helpers_dtype(dtype), max_num_seqs=3, max_prefill_tokens=16,
                                         max_seq_len=128, num_blocks=24))
            sched = Scheduler(engine.cache, chunk_size=16, stop_token_ids=[stop])
            for i, p in enumerate(prompts):
                sched.add_request(f"r{i}", p, params.max_tokens, sampling=params)
            waited = {f"r{i}": [] for i in range(3)}
            while sched.has_work():
                batch = sched.schedule_step(16, 3)
                for rid, tok in sched.commit(batch, engine.step(batch)).new_tokens.items():
                    waited[rid].append(tok)
            del engine, sched
            llm = LLM(folder, dtype=dtype, max_seq_len=128, num_blocks=24, max_running_requests=3, chunked_prefill_size=16)
            llm.scheduler._stop = frozenset([stop])
            before = llm.engine.launched_ahead
            got = llm.generate(prompts, params)
            assert got == [waited[f"r{i}"] for i in range(3)], (dtype, params)
            assert llm.engine.launched_ahead - before >= 8   # the path under test was taken
            llm.engine.cache.check()
            if dtype == "float32" and params.temperature == 0:
                cut = [w[: w.index(stop) + 1] if stop in w else w for w in want]
                assert got == cut
            del llm


def helpers_dtype(name):
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[name]


def test_captured_steps_keep_their_split_scratch_when_later_captures_need_more(tmp_path):
    """Many heads and a long maximum length: the split-KV scratch of the batch-1 step is larger than the buffer's
    first size, and the captures for larger batches need more still.  The steps captured first keep the address they
    were captured with, so that buffer has to stay alive (capturing empties the allocator's cache, which unmaps what
    was freed): the batch-1 step must still run, and give what a fresh engine without the other captures gives."""
    from prefixserve_b200 import LLM, SamplingParams
    from prefixserve_b200.config import LlamaConfig
    from prefixserve_b200.ops import tensorcore
    from prefixserve_b200.weights import write_random_model
    cfg = LlamaConfig(vocab_size=200, hidden_size=64, intermediate_size=96, num_layers=1, num_heads=32, num_kv_heads=8,
                      head_dim=64, rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None, max_position_embeddings=8192,
                      tie_word_embeddings=True)
    folder = write_random_model(tmp_path / "wide", cfg, seed=2, std=0.2, gain_noise=0.1, dtype=torch.bfloat16)
    prompt = helpers.random_tokens(200, 40, seed=4)
    params = SamplingParams(max_tokens=12, ignore_eos=True)
    # start from no scratch at all, whatever ran before in this process; what earlier engines captured stays alive here
    earlier = {key: list(held) for key, held in tensorcore._scratch.items()}
    tensorcore._scratch.clear()
    try:
        alone = LLM(folder, dtype="bfloat16", max_seq_len=8192, num_blocks=64, max_running_requests=1)
        want = alone.generate([prompt], params)
        del alone
        generations = len(next(iter(tensorcore._scratch.values()), []))
        many = LLM(folder, dtype="bfloat16", max_seq_len=8192, num_blocks=64, max_running_requests=8)
        assert len(next(iter(tensorcore._scratch.values()))) > max(generations, 1)   # the scratch did grow in between
        assert many.generate([prompt], params) == want
        many.engine.check_device_status()
        # and against the plain implementation, not only the engine against itself: the float32 logits along the
        # engine's own tokens must have those tokens at or next to the top
        plain_cfg, plain_tensors = plain_model.read_folder(folder)
        logits = plain_model.forward(plain_cfg, plain_tensors, prompt + want[0])[len(prompt) - 1: -1]
        for step, tok in enumerate(want[0]):
            assert float(logits[step, tok]) >= float(logits[step].max()) - 0.05 * float(logits[step].abs().max()), step
    finally:
        for key, held in earlier.items():
            tensorcore._scratch[key] = held + tensorcore._scratch.get(key, [])


def test_long_decode_and_first_tokens(sharp):
    """A request decoded for hundreds of steps, and the logits of the very first tokens of a sequence."""
    from prefixserve_b200.engine.replay import Replayer
    folder, (cfg, tensors) = sharp
    toks = helpers.random_tokens(helpers.TINY_B["cfg"].vocab_size, 300, seed=77)
    rp = Replayer(folder, "float32", 320)
    rows = []
    for i, t in enumerate(toks):
        rows.append(torch.from_numpy(rp.run_step({"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []})[0].copy()))
    got = torch.stack(rows)
    want = plain_model.forward(cfg, tensors, toks)
    for pos in (0, 1, 2, 15, 16, 17, 299):
        assert float((got[pos] - want[pos]).abs().max()) <= 1e-4 * float(want[pos].abs().max()), pos
    assert float((got - want).abs().max()) <= 1e-4 * float(want.abs().max())


def test_temperature_sampling_is_reproducible_and_batch_independent(sharp):
    from prefixserve_b200 import LLM, SamplingParams
    folder, _ = sharp
    prompts = prompts_b()
    sp = SamplingParams(temperature=0.9, seed=123, max_tokens=8, ignore_eos=True)
    llm = LLM(folder, dtype="float32", max_seq_len=256, num_blocks=32, max_running_requests=4, chunked_prefill_size=24)
    together = llm.generate(prompts, sp)
    alone = [llm.generate([p], sp)[0] for p in prompts]
    assert together == alone
    assert together != llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    other_seed = llm.generate(prompts, SamplingParams(temperature=0.9, seed=124, max_tokens=8, ignore_eos=True))
    assert other_seed != together


def test_command_line(sharp, tmp_path):
    folder, (cfg, tensors) = sharp
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    cmd = [sys.executable, "-m", "prefixserve_b200", "--model", str(folder), "--dtype", "float32", "--max-seq-len", "128",
           "--num-blocks", "16", "--max-running-requests", "2", "--chunked-prefill-size", "16", "--max-tokens", "5",
           "--ignore-eos", "--prompt-ids", ",".join(map(str, prompt))]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(ln) for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert lines[0]["output_ids"] == plain_model.greedy(cfg, tensors, prompt, 5)
    assert lines[1]["stats"]["num_running"] == 0


def test_engine_refuses_what_it_cannot_run(sharp):
    from prefixserve_b200.engine import Engine, EngineConfig, EngineError, StepItem
    folder, _ = sharp
    engine = Engine(EngineConfig(model_path=folder, dtype=torch.float32, max_num_seqs=2, max_prefill_tokens=16,
                                 max_seq_len=64, num_blocks=8))
    cache, runner = engine.cache, engine.runner
    slot = cache.open()
    toks = np.arange(5, dtype=np.int32)
    with pytest.raises(EngineError, match="no pages"):
        runner.step([StepItem(slot, 0, toks, (4,))])
    cache.reserve(slot, 5)
    with pytest.raises(EngineError, match="start at"):
        runner.step([StepItem(slot, 3, toks, ())])
    with pytest.raises(EngineError, match="token id"):
        runner.step([StepItem(slot, 0, toks + 100000, ())])
    with pytest.raises(EngineError, match="wanted offset"):
        runner.step([StepItem(slot, 0, toks, (5,))])
    with pytest.raises(EngineError, match="twice"):
        runner.step([StepItem(slot, 0, toks, ()), StepItem(slot, 0, toks, ())])
    with pytest.raises(EngineError, match="not open"):
        runner.step([StepItem(1, 0, toks, ())])
    assert runner.step([StepItem(slot, 0, toks, (0, 4))]).shape == (2, helpers.TINY_B["cfg"].vocab_size)
    with pytest.raises(ValueError, match="max_seq_len"):
        Engine(EngineConfig(model_path=folder, dtype=torch.float32, max_seq_len=100000, num_blocks=8))


def test_the_step_function_refuses_to_write_into_a_cached_page(sharp):
    """The debug check that is on for this whole suite (PSB200_DEBUG_CHECKS): a step may never write a position
    whose page the prefix tree owns, because another request may be reading it (the reference's harness asserts the
    same from outside, tests/test_llama_exact.py:146-151 of PrefixServe).  A slot that adopts a cached page but
    claims fewer tokens than the page holds would write into it: refused before anything is launched."""
    from prefixserve_b200.engine import Engine, EngineConfig, EngineError, StepItem
    folder, _ = sharp
    engine = Engine(EngineConfig(model_path=folder, dtype=torch.float32, max_num_seqs=2, max_prefill_tokens=32,
                                 max_seq_len=64, num_blocks=8))
    cache, runner = engine.cache, engine.runner
    assert runner.check_writes
    toks = np.arange(20, dtype=np.int32)
    first = cache.open()
    cache.reserve(first, 20)
    runner.step([StepItem(first, 0, toks, ())])
    cache.advance(first, 20)
    assert cache.publish(first, toks) == 1                      # the full page is the prefix tree's now
    matched, pages = cache.match_prefix(toks[:-1])
    assert matched == 16
    second = cache.open()
    cache.adopt(second, pages, 8)                               # wrong on purpose: the page holds 16 tokens, not 8
    cache.reserve(second, 20)
    with pytest.raises(EngineError, match="belongs to the prefix cache"):
        runner.step([StepItem(second, 8, toks[8:], ())])
    runner.check_writes = False                                 # without the check the step would have run
    cache.close(second)
    cache.close(first)
    cache.check()


def test_the_first_command_of_the_readme_runs_as_written():
    """README.md's first line: a random-weights preset, default flags (the sequence limit then follows the model's
    own 256 positions, not the 8192 the reference defaults to)."""
    readme = (ROOT / "README.md").read_text()
    line = next(ln for ln in readme.splitlines() if ln.startswith("python -m prefixserve_b200 --random-config"))
    cmd = line.split("#")[0].split()
    assert cmd[:3] == ["python", "-m", "prefixserve_b200"]
    proc = subprocess.run([sys.executable] + cmd[1:], capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(ln) for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert lines[0]["prompt_ids"] == [5, 17, 3] and len(lines[0]["output_ids"]) >= 1
    assert lines[1]["stats"]["num_running"] == 0


def test_replay_sub_command_and_per_request_stop_ids(sharp, tmp_path):
    """``python -m prefixserve_b200 replay`` is the trace program; ``--stop-token-ids`` ends a request on an id of its own."""
    folder, (cfg, tensors) = sharp
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    want = plain_model.greedy(cfg, tensors, prompt, 6)
    stop = want[3]
    cmd = [sys.executable, "-m", "prefixserve_b200", "--model", str(folder), "--dtype", "float32", "--num-blocks", "16",
           "--max-running-requests", "2", "--chunked-prefill-size", "16", "--max-tokens", "6", "--stop-token-ids", str(stop),
           "--prompt-ids", ",".join(map(str, prompt))]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = json.loads(next(ln for ln in proc.stdout.splitlines() if ln.startswith("{")))["output_ids"]
    assert got == want[: want.index(stop) + 1]
    trace = json.dumps({"step": 0, "entries": [{"id": "a", "tokens": prompt, "want": [7]}], "end": ["a"]}) + "\n"
    out = tmp_path / "out"
    cmd = [sys.executable, "-m", "prefixserve_b200", "replay", "--model", str(folder), "--dtype", "float32", "--out", str(out),
           "--max-tokens", "64"]
    proc = subprocess.run(cmd, input=trace, capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert proc.returncode == 0 and "done 0" in proc.stdout, proc.stderr[-2000:]
    row = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").copy())
    assert int(row.argmax()) == want[0]
