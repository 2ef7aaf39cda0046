"""Decode and prefill throughput of the engine on one B200, Llama-3.2-1B sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

One JSON line on stdout.  ``value`` is decoded tokens per second at batch 8
with every request's context ending at 4,096 tokens, timed on the device with
CUDA events around exactly K decode steps of the step function (sampling
kernel included, no host read-back inside the region).  ``e2e`` is the same
workload through the Python entry point (scheduler -> engine.step -> commit):
every step copies its inputs from pinned host memory and reads the sampled
tokens back.  ``prefill`` is one 2,048-token prompt in one step; ``roofline``
relates the decode step to the bytes it must read; ``points`` holds decode at
batch 1 and 64.  Weights (2.47 GB) exceed the L2 cache, so every step streams
them from HBM again.

``--impl reference`` runs PrefixServe itself (installed under baseline/_ref)
on the same model folder and workload through its own scheduler and engine.
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

MODEL = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256, "hidden_size": 2048,
    "intermediate_size": 8192, "num_hidden_layers": 16, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "max_position_embeddings": 131072, "tie_word_embeddings": True, "attention_bias": False, "mlp_bias": False,
}
FULL_LAYERS = 16
CONTEXT = 4096
PREFILL_TOKENS = 2048
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            raw = json.loads(f.read_text())
            out = {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
            if "bf16_tflops_sustained" in raw:
                out["bf16_tflops_sustained"] = float(raw["bf16_tflops_sustained"])
            return out
        except (KeyError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


# ------------------------------------------------------------------ model folder
def write_own_folder(folder: Path, layers: int, seed: int = 0, model: dict | None = None) -> None:
    """The engine's random-weights mode: config.json + model.safetensors, N(0, 0.02) bfloat16, drawn on the GPU."""
    import torch

    from prefixserve_b200.config import LlamaConfig
    from prefixserve_b200.weights import write_random_model
    cfg = LlamaConfig.from_dicts(dict(model or MODEL, num_hidden_layers=layers))
    write_random_model(folder, cfg, seed, std=0.02, dtype=torch.bfloat16, device="cuda")


def write_reference_folder(folder: Path, layers: int, seed: int = 0) -> None:
    """The same kind of folder for the reference arm, written with torch and safetensors alone: no code of this
    repository's package runs on that arm, not even to make its weights."""
    import torch
    from safetensors.torch import save_file

    cfg = dict(MODEL, num_hidden_layers=layers)
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)

    def mat(*shape):
        return (torch.randn(shape, device="cuda", generator=gen, dtype=torch.float32) * 0.02).to(torch.bfloat16).cpu()

    ones = torch.ones(h, dtype=torch.bfloat16)
    tensors = {"model.embed_tokens.weight": mat(v, h), "model.norm.weight": ones.clone()}
    for n in range(layers):
        pre = f"model.layers.{n}."
        tensors[pre + "input_layernorm.weight"] = ones.clone()
        tensors[pre + "post_attention_layernorm.weight"] = ones.clone()
        for name, shape in (("self_attn.q_proj", (q, h)), ("self_attn.k_proj", (kv, h)), ("self_attn.v_proj", (kv, h)),
                            ("self_attn.o_proj", (h, q)), ("mlp.gate_proj", (i, h)), ("mlp.up_proj", (i, h)),
                            ("mlp.down_proj", (h, i))):
            tensors[pre + name + ".weight"] = mat(*shape)
    folder.mkdir(parents=True, exist_ok=True)
    save_file(tensors, str(folder / "model.safetensors"), metadata={"format": "pt"})
    (folder / "config.json").write_text(json.dumps(cfg))


def kv_bytes_per_token(layers: int) -> int:
    return layers * 2 * MODEL["num_key_value_heads"] * MODEL["head_dim"] * 2


def prefill_flops(t: int, layers: int, prefix: int = 0) -> float:
    """Flops of a step that computes t tokens of one request over ``prefix`` cached ones and the last row's logits."""
    h, i, v = MODEL["hidden_size"], MODEL["intermediate_size"], MODEL["vocab_size"]
    q = MODEL["num_attention_heads"] * MODEL["head_dim"]
    kv = MODEL["num_key_value_heads"] * MODEL["head_dim"]
    gemm = 2.0 * t * layers * (h * (q + 2 * kv) + q * h + 3 * h * i) + 2.0 * h * v
    attn = layers * 4.0 * t * (prefix + (t + 1) / 2) * q   # QK^T and PV, causal
    return gemm + attn


def config_block(layers: int, batch: int, **more) -> dict:
    """The ``config`` of the JSON line: the same keys on both arms (flat, every size named)."""
    out = {
        "model": "Llama-3.2-1B sizes", "layers": layers, "layers_full": FULL_LAYERS, "hidden": MODEL["hidden_size"],
        "heads": MODEL["num_attention_heads"], "kv_heads": MODEL["num_key_value_heads"], "head_dim": MODEL["head_dim"],
        "intermediate": MODEL["intermediate_size"], "vocab": MODEL["vocab_size"], "tied": True,
        "global_batch": batch, "seq_len": CONTEXT, "page_size": PAGE, "prefill_tokens": PREFILL_TOKENS,
        "parallelism": "single-gpu", "l2": "inputs larger than L2 (every step reads 2.47 GB of weights)",
    }
    out.update(more)
    return out


def e2e_request_shape(batch: int, steps: int, warmup: int) -> tuple[int, int]:
    """(prompt tokens, tokens to generate) of the end-to-end workload.  Prompts are admitted two steps apart (the
    budget is one 2,048-token portion a step), so the first request has decoded about 2 * batch tokens when the last
    one starts; every request must still be alive at the last timed step and end at the benchmark's context."""
    generate = warmup + steps + 2 * batch + 4
    return CONTEXT - generate, generate


# ------------------------------------------------------------------------ clocks
class ClockSampler:
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.samples: list[list[str]] = []
        self._stop = threading.Event()
        self._proc = None
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self) -> None:
        try:
            self._proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                           "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self._proc.stdout:
                if self._stop.is_set():
                    break
                self.samples.append([c.strip() for c in line.split(",")])
        except OSError:
            pass

    def __enter__(self) -> "ClockSampler":
        self._thread.start()
        return self

    def __exit__(self, *exc) -> None:
        self._stop.set()
        if self._proc is not None:
            self._proc.terminate()

    def summary(self) -> dict:
        mhz = sorted(int(s[0]) for s in self.samples if s and s[0].isdigit())
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            for name, val in zip(names, s[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        mx = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(mhz)}


# ----------------------------------------------------------------------- own arm
def drive_e2e(engine, sched, batch: int, steps: int, warmup: int, rng, vocab: int, tag: str) -> dict:
    """``batch`` requests through scheduler -> engine.launch/finish -> commit, as the entry point's loop does (while a
    step runs, the one after it is scheduled and launched if that can be done without its tokens; every step's
    tokens are read back before its commit).  Timed by the host's clock over exactly ``steps`` full decode steps
    after ``warmup`` of them; every timed step copies its inputs from pinned host memory and reads its tokens back."""
    import numpy as np
    import torch
    runner = engine.runner
    prompt_len, generate = e2e_request_shape(batch, steps, warmup)
    for r in range(batch):
        sched.add_request(f"{tag}-{r}", rng.randint(0, vocab, size=prompt_len), generate, ignore_eos=True)
    decoding = produced = timed = 0
    t_start = None
    h2d, marks = [], []
    pending = None
    first_h2d = 0
    while (pending is not None or sched.has_work()) and timed < steps:
        if pending is None:
            pending = engine.launch(sched.schedule_step(PREFILL_TOKENS, batch))
            first_h2d = runner.last_h2d_bytes
        ahead = sched.schedule_ahead(batch)
        following = engine.launch(ahead, feed=pending) if ahead is not None else None
        work = pending.batch.work
        if all(w.end - w.start == 1 for w in work) and len(work) == batch:
            decoding += 1
            if decoding == warmup + 1:
                torch.cuda.synchronize()
                t_start = time.perf_counter()
        out = engine.finish(pending)
        if t_start is not None:
            produced += len(out)
            timed += 1
            h2d.append(runner.last_h2d_bytes if following is not None else first_h2d)
        sched.commit(pending.batch, out)
        if t_start is not None:
            marks.append(time.perf_counter())
        pending = following
        first_h2d = runner.last_h2d_bytes
    if pending is not None:
        sched.commit(pending.batch, engine.finish(pending))
    torch.cuda.synchronize()
    wall = time.perf_counter() - t_start
    for r in range(batch):
        sched.free_request(f"{tag}-{r}")
    if produced != batch * steps:
        raise RuntimeError(f"end-to-end region produced {produced} tokens in {timed} steps, not {batch} x {steps}")
    return {"value": round(produced / wall, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(sum(h2d) / max(len(h2d), 1)),
            "d2h_bytes_per_step": 4 * batch, "steps": timed, "tokens": produced, "ms_per_step": round(1e3 * wall / timed, 4),
            "ms_per_step_p50": round(1e3 * float(np.median(np.diff(marks))), 4) if len(marks) > 2 else None}


def run_own(args) -> dict:
    import numpy as np
    import torch

    from prefixserve_b200.engine import Engine, EngineConfig, Scheduler, StepItem
    from prefixserve_b200.ops import library
    from prefixserve_b200.sampling.sampler import choose_tokens

    pk = peaks()
    layers = args.layers
    work = Path(tempfile.mkdtemp(prefix="psb200-bench-"))
    try:
        write_own_folder(work, layers, model=MODEL)
        rng = np.random.RandomState(0)
        vocab = MODEL["vocab_size"]
        if args.only != "all":
            args.skip_points = True
        max_b = max(args.batch, 64 if not args.skip_points else args.batch)
        pool = max_b * (CONTEXT // PAGE) + 64
        engine = Engine(EngineConfig(model_path=work, dtype=torch.bfloat16, max_num_seqs=max_b, max_prefill_tokens=PREFILL_TOKENS,
                                     max_seq_len=CONTEXT, num_blocks=pool, page_size=PAGE, enable_prefix_cache=False,
                                     use_cuda_graphs=not args.no_graphs))
        runner, cache = engine.runner, engine.cache
        weights = engine.weight_bytes()  # what a decode step reads of them: every tensor once, the tied table once

        def sample(logits) -> None:
            if not runner.sample_in_step:  # the engine's runner chooses the tokens inside the step
                choose_tokens(logits, cache.records_dev, runner.last_row_slots)

        def fill(batch: int, upto: int) -> list[int]:
            """Opens ``batch`` requests and prefills each to ``upto`` tokens through the step function."""
            slots = []
            for _ in range(batch):
                slot = cache.open()
                at = 0
                while at < upto:
                    n = min(PREFILL_TOKENS, upto - at)
                    cache.reserve(slot, at + n)
                    runner.step([StepItem(slot, at, rng.randint(0, vocab, size=n).astype(np.int32), ())])
                    cache.advance(slot, at + n)
                    at += n
                slots.append(slot)
            return slots

        def decode_steps(slots: list[int], n: int) -> None:
            for _ in range(n):
                items = []
                for s in slots:
                    p = cache.position(s)
                    cache.reserve(s, p + 1)
                    items.append(StepItem(s, p, rng.randint(0, vocab, size=1).astype(np.int32), (0,)))
                sample(runner.step(items))
                for it in items:
                    cache.advance(it.slot, it.start + 1)

        def time_decode(batch: int, steps: int, warmup: int) -> tuple[float, int, float]:
            """ms per step (device), launches of this library's kernels in the timed region, mean context."""
            slots = fill(batch, CONTEXT - steps - warmup)
            decode_steps(slots, warmup)
            ctx_sum = sum(cache.position(s) + 1 for s in slots) * steps + batch * steps * (steps - 1) // 2
            torch.cuda.synchronize()
            before = library.launches
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            decode_steps(slots, steps)
            t1.record()
            torch.cuda.synchronize()
            launched = library.launches - before
            for s in slots:
                cache.close(s)
            return t0.elapsed_time(t1) / steps, launched, ctx_sum / (batch * steps)

        if args.only == "prefill" and args.prompt:
            # one prompt of --prompt tokens in portions of --portion, as the scheduler cuts it: device-timed, median of five
            total, portion = args.prompt, args.portion
            toks = rng.randint(0, vocab, size=total).astype(np.int32)

            def whole_prompt() -> float:
                slot = cache.open()
                cache.reserve(slot, total)
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                t0.record()
                for at in range(0, total, portion):
                    n = min(portion, total - at)
                    logits = runner.step([StepItem(slot, at, toks[at: at + n], (n - 1,) if at + n == total else ())])
                    cache.advance(slot, at + n)
                sample(logits)
                t1.record()
                torch.cuda.synchronize()
                cache.close(slot)
                return t0.elapsed_time(t1)

            with ClockSampler() as clocks:
                for _ in range(2):
                    whole_prompt()
                runs = sorted(whole_prompt() for _ in range(5))
            ms = runs[len(runs) // 2]
            flops = sum(prefill_flops(min(portion, total - at), layers, prefix=at) for at in range(0, total, portion))
            return {"only": "prefill", "prompt": total, "portion": portion, "layers": layers, "ms": round(ms, 3),
                    "value": round(total / (ms * 1e-3), 1), "tflops": round(flops / (ms * 1e-3) / 1e12, 1),
                    "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "clocks": clocks.summary()}

        if args.only == "prefill":
            torch.cuda.synchronize()
            portion = args.portion
            for _ in range(max(args.steps, 1)):
                slot = cache.open()
                cache.reserve(slot, PREFILL_TOKENS)
                for at in range(0, PREFILL_TOKENS, portion):  # the last step of the last prompt is the one profiled
                    runner.step([StepItem(slot, at, rng.randint(0, vocab, size=portion).astype(np.int32), (portion - 1,))])
                    cache.advance(slot, at + portion)
                cache.close(slot)
            torch.cuda.synchronize()
            return {"only": "prefill", "steps": args.steps, "layers": layers, "batch": 1, "weight_bytes": weights,
                    "portion": portion, "prefix": PREFILL_TOKENS - portion}

        # ---- headline: decode at the default batch, device-timed, clocks sampled meanwhile
        with ClockSampler() as clocks:
            time.sleep(0.3)
            ms_step, launches, mean_ctx = time_decode(args.batch, args.steps, args.warmup)
            time.sleep(0.3)
        value = args.batch / (ms_step * 1e-3)
        step_bytes = weights + args.batch * mean_ctx * kv_bytes_per_token(layers)
        achieved = step_bytes / (ms_step * 1e-3) / 1e9
        if args.only == "decode":
            return {"only": "decode", "value": round(value, 1), "ms_per_step": round(ms_step, 4), "layers": layers,
                    "batch": args.batch, "gpu_launches": launches, "weight_bytes": weights, "mean_context": mean_ctx,
                    "hbm_gbs": round(achieved, 1), "hbm_frac": round(achieved / pk["hbm_gbs"], 4),
                    "sizes": f"hidden {MODEL['hidden_size']}, heads {MODEL['num_attention_heads']}/{MODEL['num_key_value_heads']} of "
                             f"{MODEL['head_dim']}, vocabulary {MODEL['vocab_size']}", "clocks": clocks.summary()}

        # ---- end to end through the scheduler and engine.launch/finish (host tokens in and out)
        engine.capture_decode_graphs(range(1, max_b + 1))  # as the entry point does at start-up
        sched = Scheduler(cache, chunk_size=PREFILL_TOKENS, stop_token_ids=())
        e2e = drive_e2e(engine, sched, args.batch, args.steps, args.warmup, rng, vocab, "e2e")

        # ---- prefill: one 2,048-token prompt in one step, and the same prompt in four portions of 512
        def one_prefill(portion: int) -> float:
            slot = cache.open()
            cache.reserve(slot, PREFILL_TOKENS)
            toks = rng.randint(0, vocab, size=PREFILL_TOKENS).astype(np.int32)
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0.record()
            for at in range(0, PREFILL_TOKENS, portion):
                last = at + portion == PREFILL_TOKENS
                logits = runner.step([StepItem(slot, at, toks[at: at + portion], (portion - 1,) if last else ())])
                cache.advance(slot, at + portion)
            sample(logits)
            t1.record()
            torch.cuda.synchronize()
            cache.close(slot)
            return t0.elapsed_time(t1)

        def median_prefill(portion: int) -> float:
            for _ in range(3):
                one_prefill(portion)
            runs = sorted(one_prefill(portion) for _ in range(10))
            return runs[len(runs) // 2]

        pf_ms = median_prefill(PREFILL_TOKENS)
        flops = prefill_flops(PREFILL_TOKENS, layers)
        prefill = {"value": round(PREFILL_TOKENS / (pf_ms * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pf_ms, 4),
                   "frac": round(flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "peak": f"{pk['bf16_tflops']} TFLOP/s of {pk['source']}"}
        pc_ms = median_prefill(512)
        chunk_flops = sum(prefill_flops(512, layers, prefix=at) for at in range(0, PREFILL_TOKENS, 512))
        prefill["chunked_4x512"] = {"value": round(PREFILL_TOKENS / (pc_ms * 1e-3), 1), "ms": round(pc_ms, 4),
                                    "frac": round(chunk_flops / (pc_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

        # ---- further points: decode at batch 1 and 64, device-timed and end to end
        points = {}
        if not args.skip_points:
            for b in (1, 64):
                k = min(args.steps, 64)
                ms_b, _, ctx_b = time_decode(b, k, 3)
                points[f"decode_b{b}"] = round(b / (ms_b * 1e-3), 1)
                points[f"decode_b{b}_hbm_frac"] = round((weights + b * ctx_b * kv_bytes_per_token(layers)) / (ms_b * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
                e = drive_e2e(engine, sched, b, k, 3, rng, vocab, f"e2e-b{b}")
                points[f"e2e_decode_b{b}"] = e["value"]
                points[f"e2e_h2d_bytes_b{b}"] = e["h2d_bytes_per_step"]

        return {
            "metric": "decode tokens/s at batch 8, context 4096 (Llama-3.2-1B sizes, random weights)",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, N(0,0.02) random weights",
            "config": config_block(layers, args.batch),
            "e2e": e2e,
            "prefill": prefill,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"], "bytes_per_step": int(step_bytes),
                         "weight_bytes": int(weights)},
            "points": points,
            "clocks": clocks.summary(),
            "gpu_launches": launches,
        }
    finally:
        shutil.rmtree(work, ignore_errors=True)


# --------------------------------------------------------------- further workloads
SIZES = {"1b": "llama-3.2-1b", "3b": "llama-3.2-3b", "8b": "llama-3.1-8b"}


def _model_config(size: str) -> tuple[dict, int]:
    from prefixserve_b200.config.presets import PRESETS
    cfg = dict(PRESETS[SIZES[size]], architectures=["LlamaForCausalLM"])
    return cfg, int(cfg["num_hidden_layers"])


def run_shared_prefix(args) -> dict:
    """The multi-tenant workload the reference is named for: requests whose prompts start with one of a few long system
    prefixes, through the Python entry point (scheduler, prefix tree, chunked prefill, decode), once with the prefix
    cache and once without.  Output tokens per second of wall-clock makespan, as the reference's simulator counts."""
    import numpy as np
    import torch

    from prefixserve_b200 import LLM, SamplingParams

    cfg, full_layers = _model_config(args.model)
    layers = args.layers or full_layers
    requests, tenants, prefix_len, decode_tokens = args.requests, 4, 1024, 256
    rng = np.random.RandomState(0)
    vocab = cfg["vocab_size"]
    prefixes = [rng.randint(0, vocab, size=prefix_len).tolist() for _ in range(tenants)]
    prompts = [prefixes[r % tenants] + rng.randint(0, vocab, size=int(rng.randint(64, 513))).tolist() for r in range(requests)]
    work = Path(tempfile.mkdtemp(prefix="psb200-bench-"))
    try:
        write_own_folder(work, layers, model=cfg)
        pages = requests * (-(-(prefix_len + 512 + decode_tokens) // PAGE)) + 256
        runs = {}
        for name, enabled in (("prefix_cache", True), ("no_prefix_cache", False)):
            llm = LLM(work, dtype="bfloat16", max_seq_len=8192, num_blocks=pages, max_running_requests=min(requests, 64),
                      chunked_prefill_size=2048, enable_prefix_cache=enabled)
            llm.generate([prompts[0][:64]], SamplingParams(max_tokens=4, ignore_eos=True))  # first-use costs stay outside
            base = llm.stats()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            outs = llm.generate(prompts, SamplingParams(max_tokens=decode_tokens, ignore_eos=True))
            torch.cuda.synchronize()
            wall = time.perf_counter() - t0
            st = llm.stats()
            prompt_tokens = st.prompt_tokens - base.prompt_tokens
            cached = st.cached_prompt_tokens - base.cached_prompt_tokens
            runs[name] = {"output_tokens_per_s": round(sum(len(o) for o in outs) / wall, 1), "makespan_s": round(wall, 3),
                          "prompt_tokens": int(prompt_tokens), "prompt_tokens_computed": int(prompt_tokens - cached),
                          "prefix_hit_rate": round(cached / max(prompt_tokens, 1), 4),
                          "preemptions": int(st.preemptions - base.preemptions),
                          "steps_launched_ahead": int(llm.engine.launched_ahead)}
            del llm
            torch.cuda.empty_cache()
        on, off = runs["prefix_cache"], runs["no_prefix_cache"]
        return {
            "metric": "output tokens/s of makespan, multi-tenant shared-prefix workload through the entry point",
            "value": on["output_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic: seeded uniform-random token ids, N(0,0.02) random weights",
            "config": {"model": SIZES[args.model] + " sizes", "layers": layers, "layers_full": full_layers, "requests": requests,
                       "system_prefixes": tenants, "prefix_tokens": prefix_len, "suffix_tokens": "64-512", "decoded_tokens": decode_tokens,
                       "max_seq_len": 8192, "page_size": PAGE, "pages": pages, "chunk_budget": 2048},
            "prefix_cache": on, "no_prefix_cache": off,
            "speedup_from_prefix_cache": round(on["output_tokens_per_s"] / max(off["output_tokens_per_s"], 1e-9), 3),
        }
    finally:
        shutil.rmtree(work, ignore_errors=True)


def run_mixed(args) -> dict:
    """Steps that carry a 512-token prompt portion beside single decoded tokens of 64 requests at a long context:
    the step function's general path (no graph), device-timed."""
    import numpy as np
    import torch

    from prefixserve_b200.engine import Engine, EngineConfig, StepItem
    from prefixserve_b200.sampling import SamplingParams
    from prefixserve_b200.sampling.sampler import choose_tokens

    pk = peaks()
    cfg, full_layers = _model_config(args.model)
    layers = args.layers or full_layers
    decodes, chunk, context = args.batch if args.batch != 8 else 64, 512, args.context
    rng = np.random.RandomState(0)
    vocab = cfg["vocab_size"]
    work = Path(tempfile.mkdtemp(prefix="psb200-bench-"))
    try:
        write_own_folder(work, layers, model=cfg)
        steps, warmup = min(args.steps, 16), 3
        pages = (decodes + 1) * (context // PAGE) + 64
        engine = Engine(EngineConfig(model_path=work, dtype=torch.bfloat16, max_num_seqs=decodes + 1, max_prefill_tokens=2048,
                                     max_seq_len=context, num_blocks=pages, page_size=PAGE, enable_prefix_cache=False))
        runner, cache = engine.runner, engine.cache
        start = context - (steps + warmup) - 1
        slots = []
        for _ in range(decodes):  # the decoding requests, prefilled through the step function
            slot, at = cache.open(), 0
            while at < start:
                n = min(2048, start - at)
                cache.reserve(slot, at + n)
                runner.step([StepItem(slot, at, rng.randint(0, vocab, size=n).astype(np.int32), ())])
                cache.advance(slot, at + n)
                at += n
            slots.append(slot)
        prompt = cache.open()  # the request whose prompt arrives in portions; it starts over when it is full
        greedy = SamplingParams()

        def one_step() -> None:
            nonlocal prompt
            at = cache.position(prompt)
            if at + chunk > context:
                cache.close(prompt)
                prompt, at = cache.open(), 0
            items = [StepItem(prompt, at, rng.randint(0, vocab, size=chunk).astype(np.int32), ())]
            cache.reserve(prompt, at + chunk)
            for s in slots:
                p = cache.position(s)
                cache.reserve(s, p + 1)
                items.append(StepItem(s, p, rng.randint(0, vocab, size=1).astype(np.int32), (0,)))
            logits = runner.step(items)
            if not runner.sample_in_step:  # the engine's runner chooses the tokens inside the step
                choose_tokens(logits, cache.records_dev, runner.last_row_slots)
            for it in items:
                cache.advance(it.slot, it.start + len(it.tokens))

        for _ in range(warmup):
            one_step()
        torch.cuda.synchronize()
        portion_context = cache.position(prompt)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.perf_counter()
        t0.record()
        for _ in range(steps):
            one_step()
        t1.record()
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - w0) * 1e3 / steps
        ms = t0.elapsed_time(t1) / steps
        h, i = cfg["hidden_size"], cfg["intermediate_size"]
        q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
        per_layer = (q + 2 * kv) * h + h * q + 3 * h * i
        weights = 2 * (vocab * h + layers * per_layer)
        kv_token = layers * 2 * kv * 2
        bytes_step = weights + decodes * (context - steps // 2) * kv_token
        flops = 2.0 * chunk * layers * per_layer + layers * 4.0 * chunk * (portion_context + chunk / 2) * q
        bound_ms = max(bytes_step / (pk["hbm_gbs"] * 1e9), flops / (pk["bf16_tflops"] * 1e12)) * 1e3
        return {
            "metric": "tokens/s of steps that mix a 512-token prompt portion with single decoded tokens",
            "value": round((decodes + chunk) / (ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
            "ms_per_step": round(ms, 3), "ms_per_step_wall": round(wall_ms, 3), "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic: seeded uniform-random token ids, N(0,0.02) random weights",
            "config": {"model": SIZES[args.model] + " sizes", "layers": layers, "layers_full": full_layers, "decoding_requests": decodes,
                       "portion_tokens": chunk, "context": context, "page_size": PAGE},
            "roofline": {"bound": "max(bytes/hbm, portion flops/peak)", "ms": round(bound_ms, 3), "frac": round(bound_ms / ms, 4),
                         "of": pk["source"], "bytes_per_step": int(bytes_step), "flops_per_step": flops},
        }
    finally:
        shutil.rmtree(work, ignore_errors=True)


# ----------------------------------------------------------------- reference arm
def run_reference(args) -> dict:
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "prefixserve").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref holds no install of the reference"}
    sys.path.insert(0, str(ref))
    try:
        import numpy as np
        import torch
        from prefixserve.llama_engine import EngineConfig, LlamaEngine
        from prefixserve.scheduler import Scheduler
    except Exception as e:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"the reference does not import here: {type(e).__name__}: {e}"[:300]}

    work = Path(tempfile.mkdtemp(prefix="psb200-bench-ref-"))
    try:
        write_reference_folder(work, FULL_LAYERS)
        rng = np.random.RandomState(0)
        vocab = MODEL["vocab_size"]
        pool = args.batch * (CONTEXT // PAGE) + 64
        engine, attention, why = None, None, []
        for attention in ("flashinfer", "torch"):  # its default first, then its own other backend
            try:
                engine = LlamaEngine(EngineConfig(model_path=work, dtype=torch.bfloat16, attention=attention,
                                                  max_num_seqs=args.batch, max_prefill_tokens=PREFILL_TOKENS,
                                                  max_seq_len=CONTEXT, num_blocks=pool))
                sched = Scheduler(engine.num_blocks, chunk_size=PREFILL_TOKENS, enable_prefix_cache=False)
                sched.add_request("probe", rng.randint(0, vocab, size=40), 2, ignore_eos=True)
                while sched.has_work():
                    b = sched.schedule_step(PREFILL_TOKENS, args.batch)
                    sched.commit(b, engine.step(b))
                break
            except Exception as e:  # noqa: BLE001
                why.append(f"{attention}: {type(e).__name__}: {str(e)[:120]}")
                engine = None
        if engine is None:
            return {"impl": "reference", "unavailable": "; ".join(why)[:400]}

        prompt_len, generate = e2e_request_shape(args.batch, args.steps, args.warmup)
        sched = Scheduler(engine.num_blocks, chunk_size=PREFILL_TOKENS, enable_prefix_cache=False)
        for r in range(args.batch):
            sched.add_request(f"r{r}", rng.randint(0, vocab, size=prompt_len), generate, ignore_eos=True)
        decoding = produced = steps = 0
        t_start = None
        h2d = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler() as clocks:
            while sched.has_work() and steps < args.steps:
                batch = sched.schedule_step(PREFILL_TOKENS, args.batch)
                is_decode = all(w.end - w.start == 1 for w in batch.work) and len(batch.work) == args.batch
                if is_decode:
                    decoding += 1
                    if decoding == args.warmup + 1:
                        torch.cuda.synchronize()
                        e0.record()
                        t_start = time.perf_counter()
                out = engine.step(batch)
                if t_start is not None:
                    produced += len(out)
                    steps += 1
                    # the int32 words its engine lays out in its one pinned buffer and copies (llama_engine.py:152-227
                    # of PrefixServe): ids and positions per token, two offset arrays, last-page lengths, the rows to
                    # sample, and every request's whole page list
                    t, b = sum(w.end - w.start for w in batch.work), len(batch.work)
                    h2d.append(4 * (2 * t + 2 * (b + 1) + b + len(out) + sum(-(-w.end // PAGE) for w in batch.work)))
                sched.commit(batch, out)
            e1.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - t_start
        if produced != args.batch * args.steps:
            raise RuntimeError(f"end-to-end region produced {produced} tokens in {steps} steps, not {args.batch} x {args.steps}")
        dev_ms = e0.elapsed_time(e1)
        return {
            "impl": "reference", "metric": "decode tokens/s at batch 8, context 4096 (Llama-3.2-1B sizes, random weights)",
            "value": round(produced / (dev_ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
            "ms_per_step": round(dev_ms / max(steps, 1), 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, N(0,0.02) random weights",
            "config": config_block(FULL_LAYERS, args.batch),
            "e2e": {"value": round(produced / wall, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(sum(h2d) / max(len(h2d), 1)),
                    "d2h_bytes_per_step": 8 * args.batch, "steps": steps, "tokens": produced},
            "clocks": clocks.summary(), "attention_backend": attention, "notes": "; ".join(why),
        }
    finally:
        shutil.rmtree(work, ignore_errors=True)


def run_timeline(args) -> dict:
    """--only decode|prefill under the torch profiler: when every kernel of the last step started and ended on the
    device (also inside a replayed CUDA graph, which a launch list under ncu serialises and so cannot show).  A
    kernel's "serial" time is its end minus the latest end before it: what it adds to the step, waits included."""
    import re
    import tempfile as tf

    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        base = run_own(args)
    with tf.TemporaryDirectory() as tmp:
        trace = Path(tmp) / "trace.json"
        prof.export_chrome_trace(str(trace))
        events = json.loads(trace.read_text())["traceEvents"]
    kernels = sorted((e for e in events if e.get("cat") == "kernel"), key=lambda e: e["ts"])
    first = [i for i, e in enumerate(kernels) if "embedding_kernel" in e["name"]]
    if not first:
        return {**base, "timeline": "no step found in the trace"}
    last = first[-1]
    if args.only == "decode":  # the timed steps end with the sampling kernels; the last complete step
        ends = [i for i, e in enumerate(kernels) if "sample_finish" in e["name"]]
        last = max(i for i in first if any(j > i for j in ends))
        step = kernels[last: min(j for j in ends if j > last) + 1]
    else:
        step = kernels[last:]

    def short(name: str) -> str:
        m = re.search(r"(\w+_kernel)(<[^>]*>)?", name)
        return (m.group(1) + (m.group(2) or "")) if m else name[:48]

    t0 = prev_end = step[0]["ts"]
    rows: dict[str, list] = {}
    for e in step:
        end = e["ts"] + e["dur"]
        row = rows.setdefault(short(e["name"]), [0, 0.0])
        row[0] += 1
        row[1] += max(end - prev_end, 0.0)
        prev_end = max(prev_end, end)
    costs = kernel_costs(base) if args.profile else []
    pk = peaks()
    table = []
    for k, (n, t) in sorted(rows.items(), key=lambda kv: -kv[1][1]):
        row = {"kernel": k, "launches": n, "serial_us_each": round(t / n, 2), "serial_us_total": round(t, 1)}
        for pattern, nbytes, flops in costs:
            if re.search(pattern, k):
                bound_us = max(nbytes / (pk["hbm_gbs"] * 1e9), flops / (pk["bf16_tflops"] * 1e12)) * 1e6
                row.update({"bytes": int(nbytes), "flops": int(flops), "bound": "hbm" if nbytes / (pk["hbm_gbs"] * 1e9) >= flops / (pk["bf16_tflops"] * 1e12) else "tensor",
                            "bound_us": round(bound_us, 1), "frac_of_" + pk["source"] + "_peak": round(bound_us / t, 3) if t else None})
                break
        table.append(row)
    return {**base, "step_span_us": round(prev_end - t0, 1), "kernels_in_step": len(step), "timeline": table}


def kernel_costs(base: dict) -> list[tuple[str, float, float]]:
    """(pattern of a kernel's name, bytes it has to move, flops it has to do) for all launches of that kernel in one
    step of the profiled workload, from the model's sizes: weights once per use, the cache of the live requests,
    activations where they are the bulk.  A name that serves several products carries their sum."""
    h, i, v = MODEL["hidden_size"], MODEL["intermediate_size"], MODEL["vocab_size"]
    d, hq = MODEL["head_dim"], MODEL["num_attention_heads"]
    q, kv = hq * d, MODEL["num_key_value_heads"] * d
    layers = base["layers"]
    if base.get("only") == "decode":
        b, ctx = base["batch"], base["mean_context"]
        return [
            (r"gemm_stream_norm_kernel<.*true>", layers * 2.0 * (q + 2 * kv) * h, layers * 2.0 * b * (q + 2 * kv) * h),
            (r"gemm_stream_norm_kernel<\d+, 2,", layers * 2.0 * 2 * i * h, layers * 2.0 * b * 2 * i * h),
            (r"gemm_stream_norm_kernel<.*float", 2.0 * v * h + 4.0 * b * v, 2.0 * b * v * h),
            (r"gemm_stream_kernel", layers * 2.0 * (h * q + h * i), layers * 2.0 * b * (h * q + h * i)),
            (r"attention_decode(_tma)?_kernel", layers * b * ctx * 2.0 * kv * 2, layers * 4.0 * b * ctx * q),
            (r"sample_kernel", 4.0 * b * v, 0.0),
        ]
    t, prefix = base.get("portion", PREFILL_TOKENS), base.get("prefix", 0)
    return [
        # the projection that rotates in its epilogue has a non-zero second template argument; the other three share a name
        (r"gemm_tcgen05_kernel<\d+, [1-9]", layers * 2.0 * h * (q + 2 * kv), 2.0 * t * layers * h * (q + 2 * kv)),
        (r"gemm_tcgen05_kernel", layers * 2.0 * (q * h + 3 * h * i), 2.0 * t * layers * (q * h + 3 * h * i)),
        (r"attention_prefill_tcgen05_kernel", layers * 2.0 * (t * 2 * q + (prefix + t) * 2 * kv), layers * 4.0 * t * (prefix + (t + 1) / 2) * q),
        (r"add_rmsnorm_kernel", (2 * layers) * 12.0 * t * h, 0.0),
        (r"gemm_stream_norm_kernel<.*float", 2.0 * v * h, 2.0 * v * h),
        (r"embedding_kernel", 6.0 * t * h, 0.0),
    ]


def _no_device(args) -> bool:
    """Neither arm has a CPU path: without a CUDA device, one line says so instead of a stack of CUDA errors."""
    import torch
    if torch.cuda.is_available():
        return False
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "no CUDA device on this machine"}))
    else:
        print(json.dumps({"error": "no CUDA device on this machine; the engine has no CPU path"}))
    return True


def main() -> int:
    global MODEL, FULL_LAYERS, CONTEXT  # --only decode may be asked for other sizes and contexts
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=128)
    p.add_argument("--warmup", type=int, default=8)
    p.add_argument("--impl", choices=["own", "reference"], default="own")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the full model (recorded in config)")
    p.add_argument("--skip-points", action="store_true", help="leave out the batch-1 and batch-64 points")
    p.add_argument("--only", choices=["all", "decode", "prefill"], default="all",
                   help="decode: only the device-timed decode steps; prefill: only the 2,048-token prefill (for profilers)")
    p.add_argument("--portion", type=int, default=PREFILL_TOKENS, choices=[256, 512, 1024, 2048],
                   help="with --only prefill: the 2,048-token prompt arrives in portions of this size")
    p.add_argument("--no-graphs", action="store_true", help="run decode steps without CUDA graphs (kernel launch lists)")
    p.add_argument("--timeline", action="store_true",
                   help="with --only decode|prefill: start and end of every kernel of the last step, from the torch profiler "
                        "(numbers of a profiled run are not bench values)")
    p.add_argument("--profile", action="store_true",
                   help="--timeline plus, per kernel, the bytes and flops it has to do in the step and the fraction of the "
                        "measured peak that its time inside the step amounts to")
    p.add_argument("--workload", choices=["decode", "shared-prefix", "mixed"], default="decode",
                   help="decode: the headline line.  shared-prefix: 64 requests over 4 system prefixes through the entry "
                        "point, prefix cache on and off.  mixed: steps of one 512-token prompt portion beside 64 decoded tokens")
    p.add_argument("--model", choices=sorted(SIZES), default=None,
                   help="layer sizes for --workload shared-prefix (8b) / mixed (3b), and for --only decode (the headline stays 1b)")
    p.add_argument("--requests", type=int, default=64, help="requests of --workload shared-prefix")
    p.add_argument("--prompt", type=int, default=None,
                   help="with --only prefill: time one prompt of this many tokens, cut into portions of --portion "
                        "(--context must be at least as long)")
    p.add_argument("--context", type=int, default=None,
                   help="context of --workload mixed (8192 unless given) and of --only decode (the headline stays 4096)")
    args = p.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.prompt and (args.only != "prefill" or args.impl != "own" or (args.context or CONTEXT) < args.prompt):
        print(json.dumps({"unsupported": "--prompt goes with --only prefill of this engine and a --context at least as long"}))
        return 2
    if args.workload == "decode" and args.impl == "own" and (args.model or args.context) and \
            (args.only == "decode" or (args.only == "prefill" and args.prompt)):
        # further sizes and context lengths for the device-timed decode steps and prompts; the headline line is not touched
        if args.model:
            MODEL, full = _model_config(args.model)
            args.layers = full if args.layers == FULL_LAYERS and "--layers" not in sys.argv else args.layers
            FULL_LAYERS = full
        CONTEXT = args.context or CONTEXT
    elif args.workload == "decode" and (args.model or args.context):
        print(json.dumps({"unsupported": "--model and --context go with --only decode, --only prefill --prompt N, --workload shared-prefix or --workload mixed"}))
        return 2
    args.context = args.context or 8192
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"unsupported": f"this engine runs on one GPU; --gpus {args.gpus} is not built", "n_gpus": args.gpus}))
        return 2
    if args.workload != "decode":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference arm runs the headline workload only"}))
            return 0
        if _no_device(args):
            return 1
        args.model = args.model or ("8b" if args.workload == "shared-prefix" else "3b")
        args.layers = None if args.layers == FULL_LAYERS and "--layers" not in sys.argv else args.layers
        result = run_shared_prefix(args) if args.workload == "shared-prefix" else run_mixed(args)
    else:
        args.timeline = args.timeline or args.profile
        if args.timeline and (args.impl != "own" or args.only == "all"):
            print(json.dumps({"unsupported": "--timeline/--profile need --only decode or --only prefill of this engine"}))
            return 2
        if _no_device(args):
            return 0 if args.impl == "reference" else 1
        result = run_reference(args) if args.impl == "reference" else (run_timeline(args) if args.timeline else run_own(args))
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
