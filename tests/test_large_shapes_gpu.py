"""The layer sizes the benchmark runs (hidden 2,048, 32 query and 8 key/value heads of 64, feed-forward 8,192,
vocabulary 128,256), two layers deep, and steps with dozens of live requests: compared with the plain implementation
(on the GPU in float32, no reduced-precision matrix mode) under every cutting, in float32 and in bfloat16."""

import pytest
import torch

import helpers
import plain_model

pytestmark = pytest.mark.gpu

LENGTHS = [3, 77, 150, 210]


def config_1b(layers: int = 2):
    from prefixserve_b200.config import Llama3RopeScaling, LlamaConfig
    return LlamaConfig(vocab_size=128256, hidden_size=2048, intermediate_size=8192, num_layers=layers, num_heads=32,
                       num_kv_heads=8, head_dim=64, rms_norm_eps=1e-5, rope_theta=500000.0,
                       rope_scaling=Llama3RopeScaling(32.0, 1.0, 4.0, 8192), max_position_embeddings=131072,
                       tie_word_embeddings=True)


@pytest.fixture(scope="module")
def big(tmp_path_factory):
    from prefixserve_b200.weights import write_random_model
    torch.backends.cuda.matmul.allow_tf32 = False
    folder = write_random_model(tmp_path_factory.mktemp("llama1b2"), config_1b(), seed=7, std=0.02, gain_noise=0.05,
                                dtype=torch.bfloat16)
    cfg, tensors = plain_model.read_folder(folder)
    on_gpu = {k: v.cuda() for k, v in tensors.items()}
    return folder, cfg, on_gpu


def sequences(lengths=LENGTHS, seed=300):
    return {f"r{i}": helpers.random_tokens(128256, n, seed=seed + i) for i, n in enumerate(lengths)}


def thin(steps, keep):
    """The same trace asking only for the logits of positions where keep(request, position) holds: a row of this
    vocabulary is half a megabyte."""
    pos: dict[str, int] = {}
    out = []
    for st in steps:
        entries = []
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            entries.append(dict(e, want=[w for w in e["want"] if keep(e["id"], base + w)]))
            pos[e["id"]] = base + len(e["tokens"])
        out.append(dict(st, entries=entries))
    return out


@pytest.fixture(scope="module")
def replayers(big):
    from prefixserve_b200.engine.replay import Replayer
    folder, _, _ = big
    made = {}

    def get(dtype):
        if dtype not in made:
            made[dtype] = Replayer(folder, dtype, 1536, max_live=8)
        return made[dtype]
    return get


def run(rp, steps):
    outputs = {}
    for st in steps:
        out = rp.run_step(st)
        if out is not None:
            outputs[st["step"]] = torch.from_numpy(out.copy())
    rp.cache.check()
    assert rp.cache.free_pages(0) == rp.cache.num_pages(0)
    return helpers.collect(steps, outputs)


TRACES = {"whole": helpers.trace_whole, "tail_decode": helpers.trace_tail_decode, "portions": helpers.trace_portions,
          "mixed": helpers.trace_mixed}


@pytest.fixture(scope="module")
def truth(big):
    _, cfg, tensors = big
    out = {}
    for rid, toks in sequences().items():
        f32 = plain_model.forward(cfg, tensors, toks, device="cuda")
        b16 = plain_model.forward(cfg, tensors, toks, dtype=torch.bfloat16, device="cuda")
        out[rid] = (f32.cpu(), b16.cpu())
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", list(TRACES))
def test_benchmark_layer_sizes_under_every_cutting(big, replayers, truth, kind, dtype):
    seqs = sequences()
    keep = lambda rid, p: p % 6 == 0 or p >= len(seqs[rid]) - 34   # noqa: E731
    steps = thin(TRACES[kind](seqs), keep)
    rows = run(replayers(dtype), steps)
    for rid, toks in seqs.items():
        at = [p for p in range(len(toks)) if keep(rid, p)]
        got = torch.stack([rows[(rid, p)] for p in at])
        want, plain_bf16 = truth[rid][0][at], truth[rid][1][at]
        if dtype == "float32":
            err = float((got - want).abs().max())
            assert err <= 1e-4 * float(want.abs().max()), f"{kind}/{rid}: |diff| {err:.3e}"
        else:
            ours, theirs = helpers.rel_err(got, want), helpers.rel_err(plain_bf16, want)
            assert ours < 0.15 and ours <= 1.5 * theirs + 1e-3, f"{kind}/{rid}: engine {ours:.4f}, plain bf16 {theirs:.4f}"


@pytest.mark.parametrize("dtype,bug", [("float32", "rope_relative"), ("bfloat16", "kv_len_short")])
def test_benchmark_layer_sizes_notice_injected_faults(big, replayers, truth, dtype, bug):
    seqs = {"r3": sequences()["r3"]}
    keep = lambda rid, p: p >= 40 and p % 3 == 0   # noqa: E731
    rp = replayers(dtype)
    rp.runner.inject_bug = bug
    try:
        rows = run(rp, thin(helpers.trace_portions(seqs), keep))
    finally:
        rp.runner.inject_bug = None
    at = [p for p in range(len(seqs["r3"])) if keep("r3", p)]
    got = torch.stack([rows[("r3", p)] for p in at])
    want, plain_bf16 = truth["r3"][0][at], truth["r3"][1][at]
    if dtype == "float32":
        assert float((got - want).abs().max()) > 1e-3 * float(want.abs().max())
    else:
        assert helpers.rel_err(got, want) > 1.5 * helpers.rel_err(plain_bf16, want) + 1e-3


# ---------------------------------------------------------------------------------------------- dozens of live requests

def many(vocab: int, live: int, seed: int, prompt: int = 100):
    """``live`` requests whose last live + 4 tokens are decoded one by one: all are live before the first ends."""
    return {f"q{i}": helpers.random_tokens(vocab, prompt + (i * 7) % 23 + live + 4, seed=seed + i) for i in range(live)}


@pytest.mark.parametrize("decode_kernel", ["lanes", "tma"])
@pytest.mark.parametrize("live", [20, 64])
@pytest.mark.parametrize("which", ["D", "E"])
def test_steps_with_dozens_of_requests_match_plain(tmp_path, which, live, decode_kernel, monkeypatch):
    """20 and 64 requests live at once, bfloat16 weights: decode steps of 17 to 64 rows (mid-size products, the
    separate norm, rotary and activation kernels, decode attention at many requests) beside one 100-token portion."""
    from prefixserve_b200.engine.replay import Replayer
    from prefixserve_b200.ops import library, tensorcore
    # both decode attention kernels: the TMA-fed one is the engine's choice for long key ranges only
    monkeypatch.setattr(tensorcore, "TMA_DECODE_MIN_RANGE", 16 if decode_kernel == "tma" else 1 << 30)
    folder = helpers.make_folder(tmp_path / f"tiny{which}16", which, dtype=torch.bfloat16)
    cfg, tensors = plain_model.read_folder(folder)
    seqs = many(helpers.TINY[which]["cfg"].vocab_size, live, seed=500)
    steps = helpers.trace_many_live(seqs, tail=live + 4)
    assert max(len(st["entries"]) for st in steps) == live
    before = library.launch_counts.copy()
    rp = Replayer(folder, "bfloat16", helpers.peak_tokens(steps), max_live=live)
    rows = run(rp, steps)
    taken = library.launch_counts - before
    assert taken["attention_decode"] > 0 and taken["silu_mul"] > 0 and taken["rope_append"] > 0, dict(taken)
    assert (taken["attention_decode_tma"] > 0) == (decode_kernel == "tma") and library.tcgen05_status() == 0
    for rid, toks in seqs.items():
        at = sorted(p for (r, p) in rows if r == rid)
        assert at[-live:] == list(range(len(toks) - live, len(toks)))
        want = plain_model.forward(cfg, tensors, toks)[at]
        plain_bf16 = plain_model.forward(cfg, tensors, toks, dtype=torch.bfloat16)[at]
        got = torch.stack([rows[(rid, p)] for p in at])
        ours, theirs = helpers.rel_err(got, want), helpers.rel_err(plain_bf16, want)
        assert ours < 0.15 and ours <= 1.5 * theirs + 1e-3, f"{which}/{live}/{rid}: engine {ours:.4f}, plain bf16 {theirs:.4f}"


def test_sixty_four_requests_at_benchmark_layer_sizes(big):
    """The batch-64 decode step of the benchmark, at its layer sizes, against the plain implementation."""
    from prefixserve_b200.engine.replay import Replayer
    folder, cfg, tensors = big
    seqs = many(128256, 64, seed=900, prompt=40)
    steps = helpers.trace_many_live(seqs, tail=68)
    assert max(len(st["entries"]) for st in steps) == 64
    steps = thin(steps, lambda rid, p: p >= len(seqs[rid]) - 6)   # the steps in which all 64 are live
    rp = Replayer(folder, "bfloat16", helpers.peak_tokens(steps), max_live=64)
    rows = run(rp, steps)
    worst = (0.0, 0.0)
    for rid, toks in seqs.items():
        at = sorted(p for (r, p) in rows if r == rid)
        want = plain_model.forward(cfg, tensors, toks, device="cuda")[at].cpu()
        plain_bf16 = plain_model.forward(cfg, tensors, toks, dtype=torch.bfloat16, device="cuda")[at].cpu()
        got = torch.stack([rows[(rid, p)] for p in at])
        ours, theirs = helpers.rel_err(got, want), helpers.rel_err(plain_bf16, want)
        assert ours < 0.15 and ours <= 1.5 * theirs + 1e-3, f"{rid}: engine {ours:.4f}, plain bf16 {theirs:.4f}"
        worst = max(worst, (ours, theirs))
    assert worst[0] > 0


# ---- the widths of the larger presets: heads of 128, hidden 4,096, feed-forward 14,336, untied head -------------------

def config_8b_widths(layers: int = 2):
    from prefixserve_b200.config import Llama3RopeScaling, LlamaConfig
    return LlamaConfig(vocab_size=32064, hidden_size=4096, intermediate_size=14336, num_layers=layers, num_heads=32,
                       num_kv_heads=8, head_dim=128, rms_norm_eps=1e-5, rope_theta=500000.0,
                       rope_scaling=Llama3RopeScaling(8.0, 1.0, 4.0, 8192), max_position_embeddings=131072,
                       tie_word_embeddings=False)


@pytest.mark.parametrize("kind", ["portions", "mixed", "tail_decode"])
def test_layer_widths_of_the_8b_preset_in_bfloat16(tmp_path_factory, kind):
    """Two layers with the widths of Llama-3.1-8B (a smaller vocabulary keeps the plain model quick): heads of 128 on
    every attention kernel, products with K of 4,096 and 14,336, the few-row product on portions of 17 to 33 tokens."""
    from prefixserve_b200.engine.replay import Replayer
    from prefixserve_b200.ops import library
    from prefixserve_b200.weights import write_random_model
    torch.backends.cuda.matmul.allow_tf32 = False
    folder = write_random_model(tmp_path_factory.mktemp("llama8b2"), config_8b_widths(), seed=11, std=0.02, gain_noise=0.05,
                                dtype=torch.bfloat16)
    cfg, tensors = plain_model.read_folder(folder)
    on_gpu = {k: v.cuda() for k, v in tensors.items()}
    seqs = {f"r{i}": helpers.random_tokens(32064, n, seed=500 + i) for i, n in enumerate([5, 90, 170, 260])}
    keep = lambda rid, p: p % 5 == 0 or p >= len(seqs[rid]) - 34   # noqa: E731
    steps = thin(TRACES[kind](seqs), keep)
    before = library.launch_counts.copy()
    rows = run(Replayer(folder, "bfloat16", 1536, max_live=8), steps)
    ran = library.launch_counts - before
    assert library.tcgen05_status() == 0
    if kind != "tail_decode":
        assert ran["gemm_fewrows"] > 0 and ran["gemm_fewrows_rope"] > 0, ran
    for rid, toks in seqs.items():
        at = [p for p in range(len(toks)) if keep(rid, p)]
        got = torch.stack([rows[(rid, p)] for p in at])
        want = plain_model.forward(cfg, on_gpu, toks, device="cuda").cpu()[at]
        plain_bf16 = plain_model.forward(cfg, on_gpu, toks, dtype=torch.bfloat16, device="cuda").cpu()[at]
        ours, theirs = helpers.rel_err(got, want), helpers.rel_err(plain_bf16, want)
        assert ours < 0.15 and ours <= 1.5 * theirs + 1e-3, f"{kind}/{rid}: engine {ours:.4f}, plain bf16 {theirs:.4f}"
