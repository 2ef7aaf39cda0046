"""Trace replay against the plain implementation: every cutting of the work, float32 and bfloat16."""

import json
import os
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

LENGTHS = {"A": [5, 17, 33, 70], "B": [1, 16, 40, 70, 131], "C": [3, 48, 97], "D": [2, 64, 129, 300], "E": [2, 70, 140, 260]}
TRACES = {
    "whole": helpers.trace_whole,
    "tail_decode": helpers.trace_tail_decode,
    "portions": helpers.trace_portions,
    "mixed": helpers.trace_mixed,
}


def sequences(which):
    vocab = helpers.TINY[which]["cfg"].vocab_size
    return {f"r{i}": helpers.random_tokens(vocab, n, seed=100 + i) for i, n in enumerate(LENGTHS[which])}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {w: helpers.make_folder(tmp_path_factory.mktemp(f"tiny{w}"), w) for w in helpers.TINY}


@pytest.fixture(scope="module")
def truth(folders):
    """float32 plain logits of every sequence, whole."""
    out = {}
    for which, folder in folders.items():
        cfg, tensors = plain_model.read_folder(folder)
        out[which] = {rid: plain_model.forward(cfg, tensors, toks) for rid, toks in sequences(which).items()}
    return out


def replay(folder, dtype, steps, max_tokens=None, poison=False, smallest_class=None, seen=None):
    from prefixserve_b200.engine.replay import Replayer
    rp = Replayer(folder, dtype, max_tokens or helpers.peak_tokens(steps))
    if smallest_class:
        rp.runner.length_classes = rp.runner._length_classes(rp.cache.max_seq_len, smallest_class)
    rp.cache.poison_freed = poison
    if poison:
        for kv in rp.cache.kv:
            kv.fill_(float("nan"))   # pages nobody has written yet are as void as pages given back
    outputs = {}
    for st in steps:
        out = rp.run_step(st)
        if out is not None:
            outputs[st["step"]] = torch.from_numpy(out.copy())
    rp.cache.check()
    assert rp.cache.free_pages(0) == rp.cache.num_pages(0), "pages were not all given back"
    if seen is not None:
        seen["decode"] = sorted(rp.runner._graphs)
        seen["shapes"] = sorted(rp.runner._shape_graphs)
    return helpers.collect(steps, outputs)


@pytest.mark.parametrize("which", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("kind", list(TRACES))
def test_float32_matches_plain(folders, truth, which, kind):
    seqs = sequences(which)
    steps = TRACES[kind](seqs)
    rows = replay(folders[which], "float32", steps)
    assert len(rows) == sum(len(t) for t in seqs.values())
    for (rid, pos), got in sorted(rows.items()):
        want = truth[which][rid][pos]
        tol = 1e-4 * float(want.abs().max())
        err = float((got - want).abs().max())
        assert err <= tol, f"{which}/{kind}: request {rid} position {pos}: |diff| {err:.3e} > {tol:.3e}"


@pytest.mark.parametrize("which", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("kind", list(TRACES))
def test_bfloat16_close_to_float32_truth(folders, truth, which, kind):
    """bfloat16 engine vs float32 truth, judged against a plain bfloat16 run of the same weights."""
    seqs = sequences(which)
    steps = TRACES[kind](seqs)
    rows = replay(folders[which], "bfloat16", steps)
    cfg, tensors = plain_model.read_folder(folders[which])
    for rid, toks in seqs.items():
        want = truth[which][rid]
        got = torch.stack([rows[(rid, p)] for p in range(len(toks))])
        plain_bf16 = plain_model.forward(cfg, tensors, toks, dtype=torch.bfloat16)
        ours, theirs = helpers.rel_err(got, want), helpers.rel_err(plain_bf16, want)
        assert ours < 0.15 and ours <= 1.5 * theirs + 1e-3, f"{which}/{kind}/{rid}: engine {ours:.4f}, plain bf16 {theirs:.4f}"


@pytest.mark.parametrize("which", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("kind", list(TRACES))
def test_bfloat16_with_weights_stored_in_bfloat16(tmp_path, which, kind):
    """The same with a checkpoint in bfloat16: every product then runs on the bfloat16 kernels (a tensor that a
    checkpoint stores in float32 stays float32 and takes the float32 product, which is what the test above sees)."""
    folder = helpers.make_folder(tmp_path / f"tiny{which}16", which, dtype=torch.bfloat16)
    cfg, tensors = plain_model.read_folder(folder)
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    seqs = sequences(which)
    rows = replay(folder, "bfloat16", TRACES[kind](seqs))
    for rid, toks in seqs.items():
        want = plain_model.forward(cfg, tensors, toks)
        got = torch.stack([rows[(rid, p)] for p in range(len(toks))])
        plain_bf16 = plain_model.forward(cfg, tensors, toks, dtype=torch.bfloat16)
        ours, theirs = helpers.rel_err(got, want), helpers.rel_err(plain_bf16, want)
        assert ours < 0.15 and ours <= 1.5 * theirs + 1e-3, f"{which}/{kind}/{rid}: engine {ours:.4f}, plain bf16 {theirs:.4f}"


@pytest.mark.parametrize("kind", list(TRACES))
def test_bfloat16_with_the_prefill_kernels_on_small_shapes(tmp_path, kind, monkeypatch):
    """The tcgen05 products (plain, gated, and the projection that rotates and appends in its epilogue) and tcgen05
    attention normally wait for prompt-sized work.  Here every portion that has their head size takes them, inside
    the whole engine: cache, portions cut anywhere, other requests in the batch, pages used again.  The weights are
    stored in bfloat16 (tensors stored in float32 stay so and go to the float32 product)."""
    from prefixserve_b200.ops import library, tensorcore
    folder = helpers.make_folder(tmp_path / "tinyD16", "D", dtype=torch.bfloat16)
    cfg, tensors = plain_model.read_folder(folder)
    monkeypatch.setattr(tensorcore, "TCGEN05_MIN_TILES", 1)
    monkeypatch.setattr(tensorcore, "TCGEN05_MIN_ROWS", 1)
    monkeypatch.setattr(tensorcore, "TCGEN05_PREFILL_MIN_TOKENS", 2)
    monkeypatch.setattr(tensorcore, "USE_FEWROWS", False)  # the kernel for a few dozen rows has the test below
    taken = {"projection": 0, "gated": 0}
    projection, gated = tensorcore.tcgen05_qkv_rope_bf16, tensorcore.gemm_tcgen05_gated

    def count_projection(*args, **kwargs):
        out = projection(*args, **kwargs)
        taken["projection"] += out is not None
        return out

    def count_gated(*args, **kwargs):
        taken["gated"] += 1
        return gated(*args, **kwargs)

    monkeypatch.setattr(tensorcore, "tcgen05_qkv_rope_bf16", count_projection)
    monkeypatch.setattr(tensorcore, "gemm_tcgen05_gated", count_gated)
    before = library.launches
    seqs = sequences("D")
    steps = TRACES[kind](seqs)
    rows = replay(folder, "bfloat16", steps)
    assert library.launches > before and library.tcgen05_status() == 0
    assert taken["projection"] > 0 and taken["gated"] > 0, taken   # the paths under test were taken
    for rid, toks in seqs.items():
        want = plain_model.forward(cfg, tensors, toks)
        got = torch.stack([rows[(rid, p)] for p in range(len(toks))])
        plain_bf16 = plain_model.forward(cfg, tensors, toks, dtype=torch.bfloat16)
        ours, theirs = helpers.rel_err(got, want), helpers.rel_err(plain_bf16, want)
        assert ours < 0.15 and ours <= 1.5 * theirs + 1e-3, f"D/{kind}/{rid}: engine {ours:.4f}, plain bf16 {theirs:.4f}"


@pytest.mark.parametrize("kind", ["portions", "mixed"])
def test_bfloat16_with_the_few_row_products(tmp_path, kind, monkeypatch):
    """Portions of 17 to 64 tokens take the few-row tcgen05 product (plain, gated, and the projection that rotates
    and appends) inside the whole engine: portions cut anywhere, other requests in the batch, pages used again."""
    from prefixserve_b200.ops import library, tensorcore
    folder = helpers.make_folder(tmp_path / "tinyD16", "D", dtype=torch.bfloat16)
    cfg, tensors = plain_model.read_folder(folder)
    monkeypatch.setattr(tensorcore, "FEWROWS_MAX", {"plain": 64, "gated": 64, "rope": 64})
    seqs = sequences("D")
    steps = helpers.trace_portions(seqs, sizes=(17, 40, 64, 33, 20)) if kind == "portions" else TRACES[kind](seqs)
    before = library.launch_counts.copy()
    rows = replay(folder, "bfloat16", steps)
    ran = library.launch_counts - before
    assert library.tcgen05_status() == 0
    assert ran["gemm_fewrows"] > 0 and ran["gemm_fewrows_gated"] > 0 and ran["gemm_fewrows_rope"] > 0, ran
    for rid, toks in seqs.items():
        want = plain_model.forward(cfg, tensors, toks)
        got = torch.stack([rows[(rid, p)] for p in range(len(toks))])
        plain_bf16 = plain_model.forward(cfg, tensors, toks, dtype=torch.bfloat16)
        ours, theirs = helpers.rel_err(got, want), helpers.rel_err(plain_bf16, want)
        assert ours < 0.15 and ours <= 1.5 * theirs + 1e-3, f"{kind}/{rid}: engine {ours:.4f}, plain bf16 {theirs:.4f}"


def test_cuttings_agree_in_float32(folders):
    """The same request cut four ways gives the same logits up to rounding."""
    seqs = sequences("B")
    base = replay(folders["B"], "float32", helpers.trace_whole(seqs))
    for kind in ("tail_decode", "portions", "mixed"):
        other = replay(folders["B"], "float32", TRACES[kind](seqs))
        for key, row in base.items():
            assert float((row - other[key]).abs().max()) <= 2e-5 * float(row.abs().max()), (kind, key)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["B", "D"])
def test_pages_are_reused_in_mixed_trace(folders, truth, which, dtype):
    """A pool smaller than all requests together: pages of finished requests come back to later ones.  Every page is
    filled with NaN the moment it is given back (and before its first use), so a request that reads anything but what
    it wrote itself shows at once; the logits must be those of the plain implementation."""
    seqs = sequences(which)
    steps = helpers.trace_mixed(seqs, max_live=2, seed=3)
    total = sum(-(-len(t) // 64) * 64 for t in seqs.values())
    assert helpers.peak_tokens(steps) < total  # the pool is smaller than all requests together
    from prefixserve_b200.engine.replay import Replayer
    pages_used: dict[int, set] = {}
    rp_probe = Replayer(folders[which], dtype, helpers.peak_tokens(steps))
    for st in steps:   # the same trace, watched: some page serves two requests in turn
        rp_probe.run_step(st)
        for rid, slot in rp_probe.slot_of.items():
            for pg in rp_probe.cache.page_ids(slot):
                pages_used.setdefault(pg, set()).add(rid)
    assert any(len(owners) > 1 for owners in pages_used.values()), "no page was used again"
    rows = replay(folders[which], dtype, steps, poison=True)
    cfg, tensors = plain_model.read_folder(folders[which])
    for rid, toks in seqs.items():
        got = torch.stack([rows[(rid, p)] for p in range(len(toks))])
        want = truth[which][rid]
        assert torch.isfinite(got).all(), f"{rid}: read a page it does not own"
        if dtype == "float32":
            assert float((got - want).abs().max()) <= 1e-4 * float(want.abs().max()), rid
        else:
            plain_bf16 = plain_model.forward(cfg, tensors, toks, dtype=torch.bfloat16)
            ours, theirs = helpers.rel_err(got, want), helpers.rel_err(plain_bf16, want)
            assert ours < 0.15 and ours <= 1.5 * theirs + 1e-3, (rid, ours, theirs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["tail_decode", "mixed"])
def test_captured_steps_of_every_length_class(tmp_path, kind, dtype):
    """A captured step is sized for a class of sequence lengths (powers of two).  With classes from 32 tokens up, the
    requests here grow through three or four of them while they decode: every class gets a capture of its own, a
    step is replayed from the capture of its own class, and the logits stay those of the plain model."""
    folder = helpers.make_folder(tmp_path / "tinyE16", "E", dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    cfg, tensors = plain_model.read_folder(folder)
    seqs = sequences("E")
    seen = {}
    rows = replay(folder, dtype, TRACES[kind](seqs), smallest_class=32, seen=seen)
    assert len({klass for _, klass in seen["decode"]}) >= (3 if kind == "tail_decode" else 1), seen
    for rid, toks in seqs.items():
        want = plain_model.forward(cfg, tensors, toks)
        got = torch.stack([rows[(rid, p)] for p in range(len(toks))])
        if dtype == "float32":
            assert float((got - want).abs().max()) <= 1e-4 * float(want.abs().max()), rid
        else:
            plain_bf16 = plain_model.forward(cfg, tensors, toks, dtype=torch.bfloat16)
            ours, theirs = helpers.rel_err(got, want), helpers.rel_err(plain_bf16, want)
            assert ours < 0.15 and ours <= 1.5 * theirs + 1e-3, f"{kind}/{rid}: engine {ours:.4f}, plain bf16 {theirs:.4f}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_steps_with_portions_of_every_length_class(tmp_path, dtype):
    """The same for captured steps that hold a prompt portion: one request is fed eight tokens a step and asks for
    the last of them while another decodes, so the same shape comes back step after step while both sequences grow
    through the length classes."""
    folder = helpers.make_folder(tmp_path / "tinyE16", "E", dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    cfg, tensors = plain_model.read_folder(folder)
    vocab = helpers.TINY["E"]["cfg"].vocab_size
    seqs = {"fed": helpers.random_tokens(vocab, 248, seed=7), "decoding": helpers.random_tokens(vocab, 70, seed=8)}
    steps = [{"step": 0, "entries": [{"id": "decoding", "tokens": seqs["decoding"][:39], "want": [38]}], "end": []}]
    for k in range(31):
        steps.append({"step": k + 1, "entries": [
            {"id": "fed", "tokens": seqs["fed"][8 * k: 8 * k + 8], "want": [7]},
            {"id": "decoding", "tokens": seqs["decoding"][39 + k: 40 + k], "want": [0]}], "end": ["fed", "decoding"] if k == 30 else []})
    seen = {}
    rows = replay(folder, dtype, steps, smallest_class=32, seen=seen)
    assert len({shape[0] for shape in seen["shapes"]}) >= 3, seen
    for rid, toks in seqs.items():
        places = sorted(p for r, p in rows if r == rid)
        got = torch.stack([rows[(rid, p)] for p in places])
        want = plain_model.forward(cfg, tensors, toks)[places]
        if dtype == "float32":
            assert float((got - want).abs().max()) <= 1e-4 * float(want.abs().max()), rid
        else:
            plain_bf16 = plain_model.forward(cfg, tensors, toks, dtype=torch.bfloat16)[places]
            ours, theirs = helpers.rel_err(got, want), helpers.rel_err(plain_bf16, want)
            assert ours < 0.15 and ours <= 1.5 * theirs + 1e-3, f"{rid}: engine {ours:.4f}, plain bf16 {theirs:.4f}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_program_from_the_command_line(folders, truth, tmp_path, dtype):
    """bin/trace_run as a user runs it: stdin lines, done lines, .f32 files."""
    seqs = sequences("A")
    steps = helpers.trace_mixed(seqs, seed=5)
    out = tmp_path / "out"
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folders["A"]), "--dtype", dtype, "--out", str(out),
           "--max-tokens", str(helpers.peak_tokens(steps))]
    proc = subprocess.run(cmd, input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    vocab = helpers.TINY["A"]["cfg"].vocab_size
    outputs = {}
    for s in steps:
        f = out / f"{s['step']}.f32"
        wanted = sum(len(e["want"]) for e in s["entries"])
        assert f.exists() == (wanted > 0)
        if wanted:
            outputs[s["step"]] = torch.from_numpy(np.fromfile(f, dtype="<f4").reshape(wanted, vocab).copy())
    rows = helpers.collect(steps, outputs)
    tol = 1e-4 if dtype == "float32" else 5e-2
    for (rid, pos), got in rows.items():
        want = truth["A"][rid][pos]
        assert float((got - want).abs().max()) <= tol * float(want.abs().max()), (rid, pos)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_overlapped_launches_change_nothing(folders, dtype):
    """With and without programmatic dependent launch (each kernel starting while its predecessor drains) the logits
    are bit-identical: the overlap only moves work that does not depend on the predecessor."""
    from prefixserve_b200.ops import library
    seqs = sequences("B")
    steps = helpers.trace_mixed(seqs, seed=9) + [dict(s, step=s["step"] + 1000) for s in helpers.trace_tail_decode(seqs)]
    assert library.pdl_enabled()
    try:
        with_overlap = replay(folders["B"], dtype, steps)
        library.set_pdl(False)
        without = replay(folders["B"], dtype, steps)
    finally:
        library.set_pdl(True)
    assert with_overlap.keys() == without.keys()
    for key, row in with_overlap.items():
        assert torch.equal(row, without[key]), key


@pytest.mark.parametrize("dtype,bug", [("float32", "rope_relative"), ("bfloat16", "rope_relative"), ("bfloat16", "kv_len_short")])
def test_injected_faults_are_noticed(folders, truth, dtype, bug):
    """The comparison used above must fail when the step function is given relative positions or a short key count
    (the faults PrefixServe injects in tests/test_llama_exact.py:227-241 to prove its own suite)."""
    from prefixserve_b200.engine.replay import Replayer
    seqs = {"r0": sequences("D")["r2"]}
    steps = helpers.trace_portions(seqs)
    rp = Replayer(folders["D"], dtype, helpers.peak_tokens(steps))
    rp.runner.inject_bug = bug
    outputs = {}
    for st in steps:
        out = rp.run_step(st)
        if out is not None:
            outputs[st["step"]] = torch.from_numpy(out.copy())
    rows = helpers.collect(steps, outputs)
    want = truth["D"]["r2"]  # the sequence replayed here under the name r0
    got = torch.stack([rows[("r0", p)] for p in range(len(seqs["r0"]))])
    # the acceptance rule of the tests above must reject this run
    ours = helpers.rel_err(got[20:], want[20:])
    if dtype == "float32":
        assert float((got - want).abs().max()) > 1e-2 * float(want.abs().max()), "the injected fault went unnoticed"
    else:
        cfg, tensors = plain_model.read_folder(folders["D"])
        theirs = helpers.rel_err(plain_model.forward(cfg, tensors, seqs["r0"], dtype=torch.bfloat16)[20:], want[20:])
        assert ours > 1.5 * theirs + 1e-3, f"the injected fault went unnoticed ({ours:.4f} vs plain bf16 {theirs:.4f})"
