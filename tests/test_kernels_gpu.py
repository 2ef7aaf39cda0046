"""Each kernel alone against a plain float32 torch restatement, at sizes other than the engine's."""

import math

import pytest
import torch

import plain_model

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(0)
    torch.backends.cuda.matmul.allow_tf32 = False


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,hidden", [(37, 24), (1000, 2056)])
def test_embedding(dtype, vocab, hidden):
    from prefixserve_b200 import ops
    table = torch.randn(vocab, hidden, device=DEV).to(dtype)
    ids = torch.randint(0, vocab, (19,), device=DEV, dtype=torch.int32)
    out = ops.embedding(ids, table)
    assert out.dtype == torch.float32
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden,eps", [(7, 24, 1e-5), (33, 1000, 1e-6), (3, 5120, 3e-2)])
def test_add_rmsnorm(dtype, rows, hidden, eps):
    from prefixserve_b200 import ops
    h = torch.randn(rows, hidden, device=DEV) * 3
    delta = torch.randn(rows, hidden, device=DEV).to(dtype)
    gain = 1 + 0.1 * torch.randn(hidden, device=DEV)
    total = h + delta.float()
    want = plain_model.rms_norm(total, gain, eps)
    h1 = h.clone()
    x = ops.add_rmsnorm(h1, delta, gain, eps, dtype)
    assert torch.allclose(h1, total, rtol=0, atol=0)  # the residual sum is float32 and exact
    assert torch.allclose(x.float(), want, **tol(dtype))
    # no pending output: plain norm, stream untouched
    h2 = h.clone()
    x2 = ops.add_rmsnorm(h2, None, gain, eps, dtype)
    assert torch.equal(h2, h)
    assert torch.allclose(x2.float(), plain_model.rms_norm(h, gain, eps), **tol(dtype))
    # chosen rows only: stream untouched, rows gathered
    idx = torch.tensor([rows - 1, 0, rows // 2], device=DEV, dtype=torch.int32)
    h3 = h.clone()
    x3 = ops.add_rmsnorm(h3, delta, gain, eps, dtype, rows=idx)
    assert torch.equal(h3, h)
    assert torch.allclose(x3.float(), want[idx.long()], **tol(dtype))


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (5, 70, 33), (64, 64, 16), (130, 333, 257), (3, 1000, 2048)])
@pytest.mark.parametrize("a_dtype,w_dtype,c_dtype", [
    (torch.float32, torch.float32, torch.float32),
    (torch.bfloat16, torch.bfloat16, torch.bfloat16),
    (torch.bfloat16, torch.float32, torch.bfloat16),
    (torch.bfloat16, torch.bfloat16, torch.float32),
])
def test_gemm_simt(m, n, k, a_dtype, w_dtype, c_dtype):
    from prefixserve_b200.ops.kernels import gemm_nt_simt
    a = torch.randn(m, k, device=DEV).to(a_dtype)
    w = torch.randn(n, k, device=DEV).to(w_dtype)
    want = a.double() @ w.double().t()
    got = gemm_nt_simt(a, w, c_dtype)
    scale = math.sqrt(k)
    if c_dtype == torch.float32:
        assert torch.allclose(got.double(), want, rtol=1e-5, atol=2e-6 * scale * 10)
    else:
        assert torch.allclose(got.double(), want, rtol=1e-2, atol=1e-2 * scale)


def test_gemm_simt_rows_do_not_depend_on_the_batch():
    """A row's product is bit-identical whether it is computed alone or among others."""
    from prefixserve_b200.ops.kernels import gemm_nt_simt
    a = torch.randn(77, 300, device=DEV)
    w = torch.randn(190, 300, device=DEV)
    full = gemm_nt_simt(a, w, torch.float32)
    for r in (0, 13, 76):
        assert torch.equal(gemm_nt_simt(a[r:r + 1].contiguous(), w, torch.float32)[0], full[r])


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_matches_float64(dtype):
    from prefixserve_b200 import ops
    a = torch.randn(50, 96, device=DEV).to(dtype)
    w = torch.randn(72, 96, device=DEV).to(dtype)
    got = ops.linear(a, w, out_dtype=torch.float32)
    want = a.double() @ w.double().t()
    assert torch.allclose(got.double(), want, rtol=2e-2 if dtype == torch.bfloat16 else 1e-5, atol=0.15 if dtype == torch.bfloat16 else 1e-4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("t,inter", [(5, 7), (40, 1000)])
def test_silu_mul(dtype, t, inter):
    from prefixserve_b200 import ops
    gu = (torch.randn(t, 2 * inter, device=DEV) * 3).to(dtype)
    got = ops.silu_mul(gu)
    g, u = gu.float()[:, :inter], gu.float()[:, inter:]
    assert torch.allclose(got.float(), torch.nn.functional.silu(g) * u, **tol(dtype))


def _paged_setup(dtype, lens_new, lens_old, hq, hkv, d, page, seed=0, shuffle=True):
    """Random q/k/v for items with ``old`` cached tokens and ``new`` tokens this step; pages in random order."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    b = len(lens_new)
    total_pages = sum(-(-(o + n) // page) for o, n in zip(lens_old, lens_new)) + 3
    perm = torch.randperm(total_pages, generator=g) if shuffle else torch.arange(total_pages)
    width = max(-(-(o + n) // page) for o, n in zip(lens_old, lens_new))
    table = torch.full((b, width), -1, dtype=torch.int32)
    at = 0
    for i, (o, n) in enumerate(zip(lens_old, lens_new)):
        np_ = -(-(o + n) // page)
        table[i, :np_] = perm[at:at + np_].to(torch.int32)
        at += np_
    seqs = []
    for o, n in zip(lens_old, lens_new):
        tot = o + n
        seqs.append(dict(q=torch.randn(tot, hq, d, generator=g), k=torch.randn(tot, hkv, d, generator=g),
                         v=torch.randn(tot, hkv, d, generator=g)))
    return table, seqs, total_pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page", [(4, 2, 16, 16), (3, 1, 32, 16), (5, 5, 48, 8), (8, 2, 64, 16), (2, 1, 128, 32)])
@pytest.mark.parametrize("window", [None, 19])
def test_rope_append_then_attention(dtype, hq, hkv, d, page, window):
    """rope+append writes the pages bit-exactly where they belong; attention over cached prefix + new tokens
    matches plain attention of the whole sequence.  Covers decode at a page edge, a portion over a cached
    prefix, a fresh prompt, and page tables in random order."""
    from prefixserve_b200 import ops
    lens_old = [32, 33, 0, 15, 100]
    lens_new = [1, 1, 37, 18, 2]
    table, seqs, num_pages = _paged_setup(dtype, lens_new, lens_old, hq, hkv, d, page)
    kv = torch.full((num_pages, 2, hkv, page, d), float("nan"), dtype=dtype, device=DEV)  # poison: unread pages
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d))
    max_pos = 256
    ang = torch.outer(torch.arange(max_pos).float(), inv)
    cos, sin = ang.cos().to(DEV), ang.sin().to(DEV)

    def rot(x, pos):  # float32 rotation of x [n, h, d] at positions pos
        c = torch.cat([ang[pos].cos()] * 2, -1)[:, None, :]
        s = torch.cat([ang[pos].sin()] * 2, -1)[:, None, :]
        return plain_model.apply_rope(x, c, s)

    table_dev = table.to(DEV)
    # 1. the cached prefixes arrive through the same kernel in an earlier "step"
    for phase in ("old", "new"):
        qkv_rows, positions, items = [], [], []
        for i, (s, o, n) in enumerate(zip(seqs, lens_old, lens_new)):
            lo, hi = (0, o) if phase == "old" else (o, o + n)
            if hi == lo:
                continue
            qkv_rows.append(torch.cat([s["q"][lo:hi].reshape(hi - lo, -1), s["k"][lo:hi].reshape(hi - lo, -1),
                                       s["v"][lo:hi].reshape(hi - lo, -1)], dim=1))
            positions += list(range(lo, hi))
            items += [i] * (hi - lo)
        qkv = torch.cat(qkv_rows).to(dtype).to(DEV)
        pos_dev = torch.tensor(positions, dtype=torch.int32, device=DEV)
        item_dev = torch.tensor(items, dtype=torch.int32, device=DEV)
        q_rot = ops.rope_append(qkv, pos_dev, item_dev, cos, sin, table_dev, kv, num_heads=hq, num_kv_heads=hkv,
                                head_dim=d, page_size=page, write_kv=True)
    # pages hold exactly the rotated keys / raw values, rounded once
    for i, (s, o, n) in enumerate(zip(seqs, lens_old, lens_new)):
        tot = o + n
        k_want = rot(s["k"].to(dtype).float(), torch.arange(tot)).to(dtype)
        v_want = s["v"].to(dtype)
        for p in range(tot):
            pg = int(table[i, p // page])
            assert torch.equal(kv[pg, 1, :, p % page, :].cpu(), v_want[p]), "values must be stored bit-exactly"
            assert torch.allclose(kv[pg, 0, :, p % page, :].cpu().float(), k_want[p].float(), **tol(dtype))
    # 2. attention of the new tokens
    out = ops.attention(q_rot, kv, table_dev, pos_dev, item_dev, window=window)
    at = 0
    for i, (s, o, n) in enumerate(zip(seqs, lens_old, lens_new)):
        tot = o + n
        qf = rot(s["q"].to(dtype).float(), torch.arange(tot)).to(dtype).float()
        kf = rot(s["k"].to(dtype).float(), torch.arange(tot)).to(dtype).float()
        want = plain_model.causal_attention(qf, kf, s["v"].to(dtype).float(), window=window)[o:].reshape(n, hq * d)
        got = out[at:at + n].float().cpu()
        assert torch.isfinite(got).all(), "attention read a page it should not have (poison leaked)"
        assert torch.allclose(got, want, **tol(dtype)), f"item {i}: {(got - want).abs().max()}"
        at += n


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key(dtype):
    """One key among hundreds is made to dominate; the output must be (almost) its value."""
    from prefixserve_b200 import ops
    hq, hkv, d, page, n_ctx = 4, 2, 32, 16, 700
    needle = 123
    q = torch.zeros(1, hq, d)
    q[..., 0] = 40.0
    k = torch.randn(n_ctx, hkv, d) * 0.1
    k[needle, :, 0] = 40.0
    v = torch.randn(n_ctx, hkv, d)
    pages = -(-n_ctx // page)
    table = torch.randperm(pages + 5)[:pages].to(torch.int32)[None, :].to(DEV)
    kv = torch.full((pages + 5, 2, hkv, page, d), float("nan"), dtype=dtype, device=DEV)
    for p in range(n_ctx):
        kv[table[0, p // page], 0, :, p % page] = k[p].to(dtype).to(DEV)
        kv[table[0, p // page], 1, :, p % page] = v[p].to(dtype).to(DEV)
    out = ops.attention(q.to(dtype).to(DEV), kv, table, torch.tensor([n_ctx - 1], dtype=torch.int32, device=DEV),
                        torch.zeros(1, dtype=torch.int32, device=DEV))
    want = v[needle].to(dtype).float().repeat_interleave(hq // hkv, dim=0).reshape(1, -1)
    assert torch.allclose(out.float().cpu(), want, atol=2e-2, rtol=2e-2)
    # with a window that ends just after the needle, it must vanish from the result
    out_w = ops.attention(q.to(dtype).to(DEV), kv, table, torch.tensor([n_ctx - 1], dtype=torch.int32, device=DEV),
                          torch.zeros(1, dtype=torch.int32, device=DEV), window=n_ctx - 1 - needle)
    assert not torch.allclose(out_w.float().cpu(), want, atol=0.2, rtol=0)
    out_w2 = ops.attention(q.to(dtype).to(DEV), kv, table, torch.tensor([n_ctx - 1], dtype=torch.int32, device=DEV),
                           torch.zeros(1, dtype=torch.int32, device=DEV), window=n_ctx - needle)
    assert torch.allclose(out_w2.float().cpu(), want, atol=2e-2, rtol=2e-2)


def test_sampling_greedy_and_ties():
    from prefixserve_b200 import ops
    logits = torch.randn(6, 1001, device=DEV)
    logits[2, 77] = logits[2, 500] = 50.0  # a tie: the lower index wins
    logits[3] = 0.0
    got = ops.sample(logits)
    want = torch.argmax(logits, dim=-1)
    want[2], want[3] = 77, 0
    assert got.tolist() == want.tolist()


def test_sampling_temperature_follows_the_stated_rule():
    from prefixserve_b200 import ops
    vocab = 300
    logits = torch.randn(4, vocab, device=DEV)
    temps = torch.tensor([0.7, 0.0, 1.3, 0.7], device=DEV)
    seeds = torch.tensor([5, 5, 2**40 + 3, 5], dtype=torch.int64, device=DEV)
    poss = torch.tensor([9, 9, 0, 10], dtype=torch.int32, device=DEV)
    got = ops.sample(logits, temps, seeds, poss).tolist()
    for row in range(4):
        if float(temps[row]) == 0:
            assert got[row] == int(torch.argmax(logits[row]))
            continue
        u = plain_model.gumbel_uniform(int(seeds[row]), int(poss[row]), vocab)
        score = logits[row].cpu() / float(temps[row]) - torch.log(-torch.log(u))
        assert got[row] == int(torch.argmax(score)), row
    # same (seed, position) -> same draw, whatever the batch
    alone = ops.sample(logits[:1].contiguous(), temps[:1].contiguous(), seeds[:1].contiguous(), poss[:1].contiguous())
    assert alone.tolist()[0] == got[0]


def test_sampling_large_vocabulary_uses_several_blocks_per_row():
    from prefixserve_b200 import ops
    vocab = 50021
    logits = torch.randn(3, vocab, device=DEV)
    logits[1, 40000] = logits[1, 123] = 30.0  # a tie across blocks: the lower index wins
    got = ops.sample(logits).tolist()
    assert got == [int(torch.argmax(logits[0])), 123, int(torch.argmax(logits[2]))]
    temps = torch.tensor([0.5, 0.0, 2.0], device=DEV)
    seeds = torch.tensor([1, 2, 3], dtype=torch.int64, device=DEV)
    poss = torch.tensor([4, 5, 6], dtype=torch.int32, device=DEV)
    got = ops.sample(logits, temps, seeds, poss).tolist()
    for row in (0, 2):
        u = plain_model.gumbel_uniform(int(seeds[row]), int(poss[row]), vocab)
        score = logits[row].cpu() / float(temps[row]) - torch.log(-torch.log(u))
        assert got[row] == int(torch.argmax(score))
    assert got[1] == 123


def test_sampling_distribution():
    """Over many positions the draws follow softmax(logits / T)."""
    from prefixserve_b200 import ops
    vocab, n = 8, 20000
    row = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, -2.0, 1.5, 0.2], device=DEV)
    logits = row.repeat(n, 1).contiguous()
    t = 0.8
    got = ops.sample(logits, torch.full((n,), t, device=DEV), torch.full((n,), 17, dtype=torch.int64, device=DEV),
                     torch.arange(n, dtype=torch.int32, device=DEV))
    freq = torch.bincount(got.long(), minlength=vocab).float().cpu() / n
    want = torch.softmax(row.cpu() / t, dim=-1)
    assert float((freq - want).abs().max()) < 0.015


def test_kernels_refuse_what_they_cannot_run():
    from prefixserve_b200 import ops
    from prefixserve_b200.ops import KernelError
    with pytest.raises(KernelError):
        ops.embedding(torch.zeros(3, dtype=torch.int32), torch.zeros(4, 4))  # CPU tensors
    with pytest.raises(KernelError):
        ops.silu_mul(torch.zeros(2, 7, device=DEV))  # odd width
    with pytest.raises(KernelError):
        q = torch.zeros(1, 3, 16, device=DEV)
        kv = torch.zeros(2, 2, 2, 16, 16, device=DEV)  # 3 query heads over 2 kv heads
        ops.attention(q, kv, torch.zeros(1, 1, dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                      torch.zeros(1, dtype=torch.int32, device=DEV))
    with pytest.raises(KernelError):
        q = torch.zeros(1, 2, 512, device=DEV)  # head size beyond the kernels' limit
        kv = torch.zeros(2, 2, 2, 16, 512, device=DEV)
        ops.attention(q, kv, torch.zeros(1, 1, dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                      torch.zeros(1, dtype=torch.int32, device=DEV))


# ---- the bfloat16 tensor-core attention kernels (prefill portions, split-KV decode) -----------------------


@pytest.fixture(params=["lanes", "tma"])
def decode_kernel(request, monkeypatch):
    """Both decode attention kernels: the one in which every lane copies its pieces, and the TMA-fed one (which the
    engine takes for long key ranges; here for every range)."""
    from prefixserve_b200.ops import tensorcore
    monkeypatch.setattr(tensorcore, "TMA_DECODE_MIN_RANGE", 16 if request.param == "tma" else 1 << 30)
    return request.param


class _Batch:
    """What ops.attention reads of a step: device offsets/lengths and the host copy of the items."""

    def __init__(self, lens_old, lens_new):
        from prefixserve_b200.parts import ItemView
        starts = [0]
        for n in lens_new:
            starts.append(starts[-1] + n)
        self.item_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
        self.kv_len = torch.tensor([o + n for o, n in zip(lens_old, lens_new)], dtype=torch.int32, device=DEV)
        self.items = [ItemView(slot=i, start=o, end=o + n, first_token=s)
                      for i, (o, n, s) in enumerate(zip(lens_old, lens_new, starts))]


def _fill_pages(seqs, table, lens, hkv, d, page, num_pages):
    """Pages with every position written (keys as given, already 'rotated'), everything else NaN."""
    kv = torch.full((num_pages, 2, hkv, page, d), float("nan"), dtype=torch.bfloat16)
    for i, (s, tot) in enumerate(zip(seqs, lens)):
        for p in range(tot):
            pg = int(table[i, p // page])
            kv[pg, 0, :, p % page] = s["k"][p].to(torch.bfloat16)
            kv[pg, 1, :, p % page] = s["v"][p].to(torch.bfloat16)
    return kv.to(DEV)


@pytest.mark.parametrize("hq,hkv,d,page", [(8, 2, 64, 16), (4, 4, 64, 32), (16, 2, 128, 16), (6, 2, 64, 16), (32, 1, 64, 16)])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("mix", ["decode", "prefill", "mixed"])
def test_attention_tensor_cores(hq, hkv, d, page, window, mix, decode_kernel):
    from prefixserve_b200 import ops
    lens_old, lens_new = {
        "decode": ([31, 32, 15, 700, 0, 2999], [1, 1, 1, 1, 1, 1]),           # page edges, first token, long context (split)
        "prefill": ([0, 64, 33, 0], [150, 37, 2, 1]),                         # fresh prompt, portions over cached prefixes
        "mixed": ([500, 0, 17, 250, 47], [1, 70, 1, 9, 1]),
    }[mix]
    table, seqs, num_pages = _paged_setup(torch.bfloat16, lens_new, lens_old, hq, hkv, d, page, seed=3)
    totals = [o + n for o, n in zip(lens_old, lens_new)]
    kv = _fill_pages(seqs, table, totals, hkv, d, page, num_pages)
    batch = _Batch(lens_old, lens_new)
    q = torch.cat([s["q"][o:] for s, o in zip(seqs, lens_old)]).to(torch.bfloat16).to(DEV)
    positions = torch.cat([torch.arange(o, o + n) for o, n in zip(lens_old, lens_new)]).to(torch.int32).to(DEV)
    token_item = torch.cat([torch.full((n,), i) for i, n in enumerate(lens_new)]).to(torch.int32).to(DEV)
    table_dev = table.to(DEV)
    out = ops.attention(q, kv, table_dev, positions, token_item, window=window, ctx=batch)
    slow = ops.attention(q, kv, table_dev, positions, token_item, window=window)  # the generic kernel, same inputs
    at = 0
    for i, (s, o, n) in enumerate(zip(seqs, lens_old, lens_new)):
        bf = lambda x: x.to(torch.bfloat16).float()  # noqa: E731
        want = plain_model.causal_attention(bf(s["q"]), bf(s["k"]), bf(s["v"]), window=window)[o:].reshape(n, hq * d)
        got = out[at:at + n].float().cpu()
        assert torch.isfinite(got).all(), f"item {i}: read an unwritten slot"
        assert torch.allclose(got, want, atol=2e-2, rtol=2e-2), f"item {i}: {(got - want).abs().max()}"
        assert torch.allclose(got, slow[at:at + n].float().cpu(), atol=2e-2, rtol=2e-2)
        at += n


def test_attention_tensor_cores_find_one_far_key(decode_kernel):
    """Decode over 3,000 keys split into ranges: one early key dominates; and a prompt portion whose rows each have
    their own dominant key."""
    from prefixserve_b200 import ops
    hq, hkv, d, page, n_ctx = 8, 2, 64, 16, 3000
    g = torch.Generator().manual_seed(0)
    k = torch.randn(n_ctx, hkv, d, generator=g) * 0.1
    v = torch.randn(n_ctx, hkv, d, generator=g)
    q = torch.randn(n_ctx, hq, d, generator=g) * 0.1
    needles = {n_ctx - 1: 77}
    for row in range(n_ctx - 40, n_ctx - 1):
        needles[row] = (row * 37) % (row + 1)  # any earlier (or own) position
    for row, key in needles.items():
        q[row, :, row % d] = 30.0
        k[key, :, row % d] += 30.0
    pages = -(-n_ctx // page)
    table = torch.randperm(pages + 7, generator=g)[:pages].to(torch.int32)[None, :]
    kv = _fill_pages([dict(k=k, v=v)], table, [n_ctx], hkv, d, page, pages + 7)
    bf = lambda x: x.to(torch.bfloat16).float()  # noqa: E731
    want = plain_model.causal_attention(bf(q), bf(k), bf(v)).reshape(n_ctx, hq * d)
    for old, new in ((n_ctx - 1, 1), (n_ctx - 40, 40)):
        batch = _Batch([old], [new])
        out = ops.attention(q[old:].to(torch.bfloat16).to(DEV), kv, table.to(DEV),
                            torch.arange(old, n_ctx, dtype=torch.int32, device=DEV),
                            torch.zeros(new, dtype=torch.int32, device=DEV), ctx=batch)
        assert torch.allclose(out.float().cpu(), want[old:], atol=3e-2, rtol=3e-2), (old, new)


def _rows_of_causal_attention(q_rows, first, k, v):
    """Plain float32 attention of the rows first.. of one sequence: q_rows [n, hq, D], k/v [T, hkv, D] -> [n, hq * D]."""
    n, hq, d = q_rows.shape
    group = hq // k.shape[1]
    keys, vals = k.repeat_interleave(group, dim=1), v.repeat_interleave(group, dim=1)
    scores = torch.einsum("nhd,thd->hnt", q_rows, keys) / math.sqrt(d)
    hidden = torch.arange(k.shape[0])[None, :] > (first + torch.arange(n))[:, None]
    probs = torch.softmax(scores.masked_fill(hidden[None], float("-inf")), dim=-1)
    return torch.einsum("hnt,thd->nhd", probs, vals).reshape(n, hq * d)


@pytest.mark.parametrize("hq,hkv,d", [(16, 8, 128), (32, 8, 64)])
def test_pages_beyond_four_gigabytes_of_the_pool(hq, hkv, d, decode_kernel):
    """A pool of one layer with more than 2^31 elements (what 64 requests of 16,384 tokens take at Llama-8B sizes):
    the requests' pages lie at its far end, beyond what a 32-bit element or byte offset reaches.  A decoding request
    over 9,000 keys, a prompt portion over a prefix, and a short request on the first pages; the new tokens' keys and
    values go in through the append kernel, and one early key of the long request is made to dominate its query."""
    from prefixserve_b200 import ops
    page = 16
    per_page = 2 * hkv * page * d
    num_pages = (1 << 31) // per_page + 3000
    assert num_pages * per_page > (1 << 31)
    g = torch.Generator().manual_seed(5)
    lens_old, lens_new = [8999, 700, 40], [1, 200, 1]
    totals = [o + n for o, n in zip(lens_old, lens_new)]
    pages_per = [-(-t // page) for t in totals]
    far = num_pages - 1 - torch.randperm(2900, generator=g)        # the last pages of the pool, in random order
    table = torch.full((3, max(pages_per)), -1, dtype=torch.int32)
    table[0, :pages_per[0]] = far[:pages_per[0]].to(torch.int32)
    table[1, :pages_per[1]] = far[pages_per[0]: pages_per[0] + pages_per[1]].to(torch.int32)
    table[2, :pages_per[2]] = torch.tensor([2, 0, 1], dtype=torch.int32)[:pages_per[2]]
    kv = torch.empty(num_pages, 2, hkv, page, d, dtype=torch.bfloat16, device=DEV)
    kv[:64].fill_(float("nan"))
    kv[-3000:].fill_(float("nan"))
    seqs = []
    for i, (o, t) in enumerate(zip(lens_old, totals)):
        q = torch.randn(t, hq, d, generator=g) * 0.3
        k = torch.randn(t, hkv, d, generator=g) * 0.3
        v = torch.randn(t, hkv, d, generator=g)
        if i == 0:
            q[t - 1, :, 7] = 30.0
            k[1234, :, 7] += 30.0
        seqs.append(dict(q=q.to(torch.bfloat16), k=k.to(torch.bfloat16), v=v.to(torch.bfloat16)))
        pos = torch.arange(o)
        pg = table[i, pos // page].long().to(DEV)
        kv[pg, 0, :, (pos % page).to(DEV)] = seqs[i]["k"][:o].to(DEV)
        kv[pg, 1, :, (pos % page).to(DEV)] = seqs[i]["v"][:o].to(DEV)
    # the new tokens arrive through the append kernel (angles of zero: the keys are stored as they are)
    cos = torch.ones(max(totals), d // 2, device=DEV)
    sin = torch.zeros(max(totals), d // 2, device=DEV)
    qkv = torch.cat([torch.cat([s[n][o:].reshape(t - o, -1) for n in ("q", "k", "v")], dim=1)
                     for s, o, t in zip(seqs, lens_old, totals)]).to(DEV)
    positions = torch.cat([torch.arange(o, t) for o, t in zip(lens_old, totals)]).to(torch.int32).to(DEV)
    token_item = torch.cat([torch.full((n,), i) for i, n in enumerate(lens_new)]).to(torch.int32).to(DEV)
    table_dev = table.to(DEV)
    q_rot = ops.rope_append(qkv, positions, token_item, cos, sin, table_dev, kv, num_heads=hq, num_kv_heads=hkv,
                            head_dim=d, page_size=page, write_kv=True)
    last = int(table[0, (totals[0] - 1) // page])
    assert last * per_page > (1 << 31) - 3000 * per_page
    assert torch.equal(kv[last, 1, :, (totals[0] - 1) % page].cpu(), seqs[0]["v"][-1]), "the append kernel missed its page"
    out = ops.attention(q_rot, kv, table_dev, positions, token_item, ctx=_Batch(lens_old, lens_new))
    torch.cuda.synchronize()
    at = 0
    for i, (s, o, t) in enumerate(zip(seqs, lens_old, totals)):
        want = _rows_of_causal_attention(s["q"][o:].float(), o, s["k"].float(), s["v"].float())
        got = out[at: at + t - o].float().cpu()
        assert torch.isfinite(got).all(), f"item {i} read a page that is not its own"
        assert torch.allclose(got, want, atol=3e-2, rtol=3e-2), (i, float((got - want).abs().max()))
        at += t - o
    needle = seqs[0]["v"][1234].float().repeat_interleave(hq // hkv, dim=0).reshape(-1)
    assert torch.allclose(out[0].float().cpu(), needle, atol=3e-2, rtol=3e-2), "the dominant key of the long request was missed"
    del kv
    torch.cuda.empty_cache()


@pytest.mark.parametrize("hq,hkv,d", [(24, 8, 128), (32, 8, 64)])
def test_decode_attention_with_every_sm_busy(hq, hkv, d, decode_kernel):
    """Dozens of requests with thousands of keys each, one key range per request: every SM holds several CTAs whose
    copies finish in any order.  (With heads of 128 the TMA-fed kernel once had six stages for four consumer warps, so a
    stage passed from warp to warp and a warp could take another's unfinished phase for its own: only a loaded device
    showed it.)  Compared with the generic kernel on the same pages."""
    from prefixserve_b200 import ops
    from prefixserve_b200.ops import library
    page, items = 16, 40
    g = torch.Generator().manual_seed(11)
    lens = [int(x) for x in torch.randint(1500, 4000, (items,), generator=g)]
    pages_per = [-(-n // page) for n in lens]
    num_pages = sum(pages_per) + 9
    perm = torch.randperm(num_pages, generator=g)
    table = torch.zeros(items, max(pages_per), dtype=torch.int32)
    at = 0
    for i, n in enumerate(pages_per):
        table[i, :n] = perm[at: at + n].to(torch.int32)
        at += n
    kv = (torch.randn(num_pages, 2, hkv, page, d, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    q = torch.randn(items, hq, d, generator=g).to(torch.bfloat16).to(DEV)
    batch = _Batch([n - 1 for n in lens], [1] * items)
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    token_item = torch.arange(items, dtype=torch.int32, device=DEV)
    for _ in range(3):   # several launches back to back: the second starts while the first drains
        fast = ops.attention(q, kv, table.to(DEV), positions, token_item, ctx=batch)
    slow = ops.attention(q, kv, table.to(DEV), positions, token_item)
    assert library.tcgen05_status() == 0
    assert torch.isfinite(fast.float()).all()
    assert torch.allclose(fast.float(), slow.float(), atol=2e-2, rtol=2e-2), float((fast.float() - slow.float()).abs().max())


@pytest.mark.parametrize("static_len,window", [(256, 50), (1024, 114), (512, 16), (4096, 300), (300, 290)])
def test_windowed_decode_with_the_launch_shapes_of_a_captured_step(static_len, window, decode_kernel):
    """A captured decode step is launched with key ranges sized from the engine's longest sequence, not from the
    step's own lengths.  With a window, the keys an item reads start at the 16-aligned beginning of the window, so
    their number depends on (length - window) mod 16 and reaches window + 15: the ranges must cover that for every
    length.  The newest key dominates every query here and the oldest key of the window comes second, so a range
    that stops short, or a merge that reads another item's partial results, gives another answer."""
    from prefixserve_b200.ops import tensorcore
    hq, hkv, d, page = 4, 2, 64, 16
    lengths = [k for k in range(max(1, window - 20), min(static_len, window + 70) + 1)]
    g = torch.Generator().manual_seed(1)
    longest = max(lengths)
    k = torch.randn(longest, hkv, d, generator=g) * 0.1
    v = torch.randn(longest, hkv, d, generator=g)
    pages = -(-longest // page)
    table = torch.randperm(pages + 5, generator=g)[:pages].to(torch.int32)[None, :]
    bf = lambda x: x.to(torch.bfloat16).float()  # noqa: E731
    for kvl in lengths:
        pos = kvl - 1
        q = torch.randn(1, hq, d, generator=g) * 0.1
        kk = k[:kvl].clone()
        q[0, :, pos % d] = 30.0
        kk[pos, :, pos % d] += 30.0                          # the newest key
        kk[max(0, pos - window + 1), :, pos % d] += 29.0     # the oldest key still inside the window
        if pos - window >= 0:
            kk[pos - window, :, pos % d] += 40.0             # just outside: must not be seen
        kv = _fill_pages([dict(k=kk, v=v[:kvl])], table, [kvl], hkv, d, page, pages + 5)
        batch = _Batch([kvl - 1], [1])
        out = tensorcore.attention_bf16(q.to(torch.bfloat16).to(DEV), kv, table.to(DEV), batch.item_start, batch.kv_len,
                                        [1], [kvl], window=window, scale=1.0 / math.sqrt(d), static_kv_len=static_len)
        scores = torch.einsum("hd,khd->hk", bf(q[0]), bf(kk).repeat_interleave(hq // hkv, dim=1)) / math.sqrt(d)
        scores[:, : max(0, pos - window + 1)] = float("-inf")
        want = torch.einsum("hk,khd->hd", torch.softmax(scores, -1), bf(v[:kvl]).repeat_interleave(hq // hkv, dim=1))
        got = out.float().cpu().view(hq, d)
        assert torch.allclose(got, want, atol=3e-2, rtol=3e-2), (kvl, float((got - want).abs().max()))


@pytest.mark.parametrize("hq,hkv,d,page", [(8, 2, 64, 16), (4, 4, 64, 64), (6, 2, 128, 16), (3, 1, 128, 32), (2, 1, 64, 128)])
@pytest.mark.parametrize("window", [None, 100, 300])
def test_attention_prefill_tcgen05(hq, hkv, d, page, window, monkeypatch):
    """Prompt portions of every shape on the tcgen05 kernel: whole tiles and ragged ones, over cached prefixes that end
    inside a page and inside a key block, next to two-token portions and decode tokens."""
    from prefixserve_b200 import ops
    from prefixserve_b200.ops import library, tensorcore
    monkeypatch.setattr(tensorcore, "TCGEN05_PREFILL_MIN_TOKENS", 2)
    lens_old = [0, 200, 1000, 77, 3, 640, 0]
    lens_new = [300, 513, 256, 2, 129, 1, 128]
    table, seqs, num_pages = _paged_setup(torch.bfloat16, lens_new, lens_old, hq, hkv, d, page, seed=5)
    totals = [o + n for o, n in zip(lens_old, lens_new)]
    kv = _fill_pages(seqs, table, totals, hkv, d, page, num_pages)
    batch = _Batch(lens_old, lens_new)
    q = torch.cat([s["q"][o:] for s, o in zip(seqs, lens_old)]).to(torch.bfloat16).to(DEV)
    positions = torch.cat([torch.arange(o, o + n) for o, n in zip(lens_old, lens_new)]).to(torch.int32).to(DEV)
    token_item = torch.cat([torch.full((n,), i) for i, n in enumerate(lens_new)]).to(torch.int32).to(DEV)
    out = ops.attention(q, kv, table.to(DEV), positions, token_item, window=window, ctx=batch)
    assert library.tcgen05_status() == 0, "a bounded wait in the kernel gave up"
    at = 0
    for i, (s, o, n) in enumerate(zip(seqs, lens_old, lens_new)):
        bf = lambda x: x.to(torch.bfloat16).float()  # noqa: E731
        want = plain_model.causal_attention(bf(s["q"]), bf(s["k"]), bf(s["v"]), window=window)[o:].reshape(n, hq * d)
        got = out[at:at + n].float().cpu()
        assert torch.isfinite(got).all(), f"item {i}: read an unwritten slot"
        assert torch.allclose(got, want, atol=2e-2, rtol=2e-2), f"item {i}: {(got - want).abs().max()}"
        at += n


def test_attention_prefill_tcgen05_every_row_finds_its_own_key():
    """600 new rows over 1,500 cached keys; each row has one key, anywhere before it, that must win."""
    from prefixserve_b200 import ops
    from prefixserve_b200.ops import library
    hq, hkv, d, page, n_ctx, old = 4, 2, 64, 16, 2100, 1500
    g = torch.Generator().manual_seed(1)
    k = torch.randn(n_ctx, hkv, d, generator=g) * 0.1
    v = torch.randn(n_ctx, hkv, d, generator=g)
    q = torch.randn(n_ctx, hq, d, generator=g) * 0.1
    for row in range(old, n_ctx):
        key = (row * 7919) % (row + 1)
        q[row, :, row % d] = 30.0
        k[key, :, row % d] += 30.0
    pages = -(-n_ctx // page)
    table = torch.randperm(pages + 7, generator=g)[:pages].to(torch.int32)[None, :]
    kv = _fill_pages([dict(k=k, v=v)], table, [n_ctx], hkv, d, page, pages + 7)
    bf = lambda x: x.to(torch.bfloat16).float()  # noqa: E731
    want = plain_model.causal_attention(bf(q), bf(k), bf(v)).reshape(n_ctx, hq * d)
    new = n_ctx - old
    out = ops.attention(q[old:].to(torch.bfloat16).to(DEV), kv, table.to(DEV), torch.arange(old, n_ctx, dtype=torch.int32, device=DEV),
                        torch.zeros(new, dtype=torch.int32, device=DEV), ctx=_Batch([old], [new]))
    assert library.tcgen05_status() == 0
    assert torch.allclose(out.float().cpu(), want[old:], atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("d,page", [(64, 16), (128, 32)])
@pytest.mark.parametrize("ranges,min_blocks", [(2, 1), (3, 1), (5, 2), (8, 1)])
@pytest.mark.parametrize("window", [None, 260])
def test_attention_prefill_over_several_key_ranges(d, page, ranges, min_blocks, window, monkeypatch):
    """A short portion over a long cached prefix: the keys are cut into ranges, each CTA keeps a partial result and a
    second kernel merges them.  Range counts that do not divide the number of key blocks, ranges that come out empty
    (a launch sized for a longer sequence than the step has; a window that leaves the first ranges nothing; a
    neighbouring item without a prefix), and one key per row, anywhere before it, that must win."""
    from prefixserve_b200 import ops
    from prefixserve_b200.ops import library, tensorcore
    monkeypatch.setattr(tensorcore, "TCGEN05_PREFILL_MIN_TOKENS", 2)
    monkeypatch.setattr(tensorcore, "PREFILL_MAX_KEY_RANGES", ranges)
    monkeypatch.setattr(tensorcore, "PREFILL_MIN_KEY_RANGES", 2)
    monkeypatch.setattr(tensorcore, "PREFILL_MIN_BLOCKS_PER_RANGE", min_blocks)
    hq, hkv = 4, 2
    lens_old, lens_new = [1390, 0, 700], [170, 40, 130]
    table, seqs, num_pages = _paged_setup(torch.bfloat16, lens_new, lens_old, hq, hkv, d, page, seed=21)
    for s, o, n in zip(seqs, lens_old, lens_new):
        for row in range(o, o + n):
            lo = max(0, row - window + 1) if window else 0
            key = lo + (row * 7919) % (row + 1 - lo)
            s["q"][row, :, row % d] = 30.0
            s["k"][key, :, row % d] += 30.0
    totals = [o + n for o, n in zip(lens_old, lens_new)]
    kv = _fill_pages(seqs, table, totals, hkv, d, page, num_pages)
    q = torch.cat([s["q"][o:] for s, o in zip(seqs, lens_old)]).to(torch.bfloat16).to(DEV)
    positions = torch.cat([torch.arange(o, o + n) for o, n in zip(lens_old, lens_new)]).to(torch.int32).to(DEV)
    token_item = torch.cat([torch.full((n,), i) for i, n in enumerate(lens_new)]).to(torch.int32).to(DEV)
    batch = _Batch(lens_old, lens_new)
    bf = lambda x: x.to(torch.bfloat16).float()  # noqa: E731
    for static_len in (None, 4096):
        plan = tensorcore._attention_plan(lens_new, totals, int(window or 0), hq // hkv, hkv, d, page, 148, static_len)
        assert plan["tcgen05"] and plan["kv_splits"] > 1, plan
        out = tensorcore.attention_bf16(q, kv, table.to(DEV), batch.item_start, batch.kv_len, lens_new, totals, window=window,
                                        scale=1.0 / math.sqrt(d), static_kv_len=static_len, token_item=token_item)
        assert library.tcgen05_status() == 0
        at = 0
        for i, (s, o, n) in enumerate(zip(seqs, lens_old, lens_new)):
            want = plain_model.causal_attention(bf(s["q"]), bf(s["k"]), bf(s["v"]), window=window)[o:].reshape(n, hq * d)
            got = out[at:at + n].float().cpu()
            assert torch.isfinite(got).all(), (i, static_len)
            assert torch.allclose(got, want, atol=3e-2, rtol=3e-2), (i, static_len, float((got - want).abs().max()))
            at += n


@pytest.mark.parametrize("seed", range(12))
def test_attention_tensor_cores_random_steps_agree_with_the_generic_kernel(seed, monkeypatch, decode_kernel):
    """Random steps (head counts, page sizes, windows, cached lengths, portion lengths from 1 to 700 tokens) through
    the tensor-core kernels and through the generic one-warp-per-row kernel on the same pages."""
    from prefixserve_b200 import ops
    from prefixserve_b200.ops import library, tensorcore
    import random
    rnd = random.Random(seed)
    d = rnd.choice([64, 128])
    hkv = rnd.choice([1, 2, 3])
    hq = hkv * rnd.choice([1, 2, 4, 7])
    page = rnd.choice([16, 32, 64])
    window = rnd.choice([None, None, 17, 130, 500])
    monkeypatch.setattr(tensorcore, "TCGEN05_PREFILL_MIN_TOKENS", rnd.choice([2, 64, 64]))
    n_items = rnd.randint(1, 5)
    lens_new = [rnd.choice([1, 1, 2, rnd.randint(3, 130), rnd.randint(120, 700)]) for _ in range(n_items)]
    lens_old = [rnd.choice([0, rnd.randint(1, 40), rnd.randint(100, 900)]) for _ in range(n_items)]
    table, seqs, num_pages = _paged_setup(torch.bfloat16, lens_new, lens_old, hq, hkv, d, page, seed=100 + seed)
    totals = [o + n for o, n in zip(lens_old, lens_new)]
    kv = _fill_pages(seqs, table, totals, hkv, d, page, num_pages)
    q = torch.cat([s["q"][o:] for s, o in zip(seqs, lens_old)]).to(torch.bfloat16).to(DEV)
    positions = torch.cat([torch.arange(o, o + n) for o, n in zip(lens_old, lens_new)]).to(torch.int32).to(DEV)
    token_item = torch.cat([torch.full((n,), i) for i, n in enumerate(lens_new)]).to(torch.int32).to(DEV)
    fast = ops.attention(q, kv, table.to(DEV), positions, token_item, window=window, ctx=_Batch(lens_old, lens_new))
    slow = ops.attention(q, kv, table.to(DEV), positions, token_item, window=window)
    assert library.tcgen05_status() == 0
    what = (d, hq, hkv, page, window, lens_old, lens_new)
    assert torch.isfinite(fast.float()).all(), what
    assert torch.allclose(fast.float(), slow.float(), atol=2e-2, rtol=2e-2), (what, float((fast.float() - slow.float()).abs().max()))


def test_attention_shapes_outside_the_tensor_core_kernels_fall_back():
    from prefixserve_b200.ops.tensorcore import attention_bf16_supported
    assert attention_bf16_supported(64, 16) and attention_bf16_supported(128, 64)
    assert not attention_bf16_supported(48, 16) and not attention_bf16_supported(64, 8) and not attention_bf16_supported(64, 48)


# ---- the weight-streaming product for few rows ---------------------------------------------------------------

@pytest.mark.parametrize("m", [1, 8, 13, 32, 40])
@pytest.mark.parametrize("inter,k", [(40, 64), (112, 96), (1000, 2048)])
def test_gated_linear(m, inter, k):
    """Whatever route the row count takes (streaming product, library product plus the activation kernel)."""
    from prefixserve_b200 import ops
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, device=DEV) / math.sqrt(k)).to(torch.bfloat16)
    got = ops.gated_linear(x, w)
    y = x.double() @ w.double().t()
    want = torch.nn.functional.silu(y[:, :inter]) * y[:, inter:]
    assert got.shape == (m, inter)
    assert torch.allclose(got.double(), want, rtol=3e-2, atol=3e-2)
    gelu = ops.gated_linear(x, w, "gelu_tanh")
    want = torch.nn.functional.gelu(y[:, :inter], approximate="tanh") * y[:, inter:]
    assert torch.allclose(gelu.double(), want, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("m", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(48, 64), (333, 96), (1000, 2048), (16, 8192), (5000, 512)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_stream(m, n, k, out_dtype):
    from prefixserve_b200.ops.tensorcore import gemm_stream
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = torch.randn(n, k, device=DEV).to(torch.bfloat16)
    got = gemm_stream(x, w, out_dtype)
    want = x.double() @ w.double().t()
    if out_dtype == torch.float32:
        assert torch.allclose(got.double(), want, rtol=1e-4, atol=1e-3 * math.sqrt(k))
    else:
        assert torch.allclose(got.double(), want, rtol=1e-2, atol=1e-2 * math.sqrt(k))
    alone = gemm_stream(x[m - 1:].contiguous(), w, out_dtype)
    if m <= 8:
        assert torch.equal(alone[0], got[m - 1])  # a row's sum order does not depend on the batch


@pytest.mark.parametrize("m", [1, 8, 13])
@pytest.mark.parametrize("inter,k", [(40, 64), (112, 96), (5000, 2048)])
def test_gemm_stream_gated(m, inter, k):
    from prefixserve_b200.ops.tensorcore import gemm_stream_gated
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, device=DEV) / math.sqrt(k)).to(torch.bfloat16)
    got = gemm_stream_gated(x, w)
    y = x.double() @ w.double().t()
    want = torch.nn.functional.silu(y[:, :inter]) * y[:, inter:]
    assert torch.allclose(got.double(), want, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("m", [1, 16, 17, 40, 200])
def test_float32_outputs_of_bfloat16_products_are_never_rounded_to_bfloat16(m):
    """Logits: whatever the number of rows, and so whichever kernel or library call does the product, the float32
    result carries the float32 sums (a detour through a bfloat16 result would cost 8 bits)."""
    from prefixserve_b200 import ops
    n, k = 1000, 512
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) / math.sqrt(k)).to(torch.bfloat16)
    got = ops.linear(x, w, out_dtype=torch.float32)
    want = x.double() @ w.double().t()
    assert got.dtype == torch.float32
    assert float((got.double() - want).abs().max()) <= 2e-5 * float(want.abs().max())


# ---- the streaming product with the residual sum and the RMSNorm in front of it folded in ---------------------------

def _plain_normed(h, pending, gain, eps, rows=None):
    v = h.double() + (0 if pending is None else pending.double())
    if rows is not None:
        v = v[rows.long()]
    return v, v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * gain.double()


@pytest.mark.parametrize("m", [1, 5, 8, 11, 16])
@pytest.mark.parametrize("n,k,eps", [(40, 64, 1e-5), (1000, 96, 1e-6), (3072, 2048, 1e-5), (520, 3104, 2e-3), (96, 8192, 1e-5)])
@pytest.mark.parametrize("with_pending", [True, False])
def test_norm_fused_linear(m, n, k, eps, with_pending):
    from prefixserve_b200 import ops
    from prefixserve_b200.ops.tensorcore import norm_linear_bf16
    h = torch.randn(m, k, device=DEV) * 3.0
    pending = torch.randn(m, k, device=DEV).to(torch.bfloat16) if with_pending else None
    gain = 1.0 + 0.3 * torch.randn(k, device=DEV)
    w = (torch.randn(n, k, device=DEV) / math.sqrt(k)).to(torch.bfloat16)
    x = ops.NormedRows(h.clone(), pending, gain, eps, torch.bfloat16)
    got = norm_linear_bf16(x, w, torch.float32)
    if m > 8 and k > 4096:
        assert got is None  # beyond the kernel: the caller takes the unfused way
        got = ops.linear(x, w, out_dtype=torch.float32)
    v, normed = _plain_normed(h, pending, gain, eps)
    want = normed @ w.double().t()
    assert float((got.double() - want).abs().max()) <= 2e-2 * float(want.abs().max()) + 1e-3
    assert torch.allclose(x.residual().double(), v, rtol=0, atol=1e-6)   # the float32 stream after the sum: exact
    # the unfused way, through the norm's own kernel, for comparison of the error against float64
    y = ops.NormedRows(h.clone(), pending, gain, eps, torch.bfloat16)
    unfused = ops.linear(y.tensor(), w, out_dtype=torch.float32)
    err_fused, err_unfused = float((got.double() - want).abs().max()), float((unfused.double() - want).abs().max())
    assert err_fused <= 2.0 * err_unfused + 1e-3 * float(want.abs().max())


def test_norm_fused_linear_on_chosen_rows_and_gated(monkeypatch):
    from prefixserve_b200 import ops
    from prefixserve_b200.ops import tensorcore
    from prefixserve_b200.ops.tensorcore import norm_gated_linear_bf16, norm_linear_bf16
    monkeypatch.setattr(tensorcore, "STREAM_M", 16)  # the kernels' own limit (the engine hands 9 rows and more to another kernel)
    t, k, n, eps = 37, 160, 1031, 1e-5
    h = torch.randn(t, k, device=DEV)
    pending = torch.randn(t, k, device=DEV).to(torch.bfloat16)
    gain = 1.0 + 0.3 * torch.randn(k, device=DEV)
    w = (torch.randn(n, k, device=DEV) / math.sqrt(k)).to(torch.bfloat16)
    rows = torch.tensor([36, 0, 7, 7, 19], dtype=torch.int32, device=DEV)
    before = h.clone()
    x = ops.NormedRows(h, pending, gain, eps, torch.bfloat16, rows)
    got = norm_linear_bf16(x, w, torch.float32)
    assert got is not None and torch.equal(h, before)           # a row selection leaves the stream alone
    _, normed = _plain_normed(before, pending, gain, eps, rows)
    want = normed @ w.double().t()
    assert float((got.double() - want).abs().max()) <= 2e-2 * float(want.abs().max())
    assert torch.equal(got[2], got[3])
    for m, inter, kk in [(3, 72, 64), (16, 1000, 2048), (8, 333, 4128)]:
        h = torch.randn(m, kk, device=DEV)
        pending = torch.randn(m, kk, device=DEV).to(torch.bfloat16)
        gain = 1.0 + 0.3 * torch.randn(kk, device=DEV)
        w = (torch.randn(2 * inter, kk, device=DEV) / math.sqrt(kk)).to(torch.bfloat16)
        x = ops.NormedRows(h.clone(), pending, gain, eps, torch.bfloat16)
        act = norm_gated_linear_bf16(x, w)
        assert act is not None and act.dtype == torch.bfloat16
        v, normed = _plain_normed(h, pending, gain, eps)
        y = (normed @ w.double().t()).to(torch.bfloat16).double()
        want = torch.nn.functional.silu(y[:, :inter]) * y[:, inter:]
        assert float((act.double() - want).abs().max()) <= 3e-2 * float(want.abs().max()) + 3e-2
        assert torch.allclose(x.residual().double(), v, rtol=0, atol=1e-6)


@pytest.mark.parametrize("lens_new,lens_old", [([130], [0]), ([64, 1, 70, 3], [5, 40, 0, 17]), ([300, 45], [16, 31])])
@pytest.mark.parametrize("hq,hkv,d,page,k", [(8, 2, 64, 16, 512), (3, 1, 48, 8, 96), (4, 4, 128, 32, 2048), (6, 2, 128, 16, 520)])
@pytest.mark.parametrize("rotate", [True, False])
@pytest.mark.parametrize("width", [0, 128, 256])
def test_projection_of_many_tokens_rotates_and_appends_in_its_epilogue(monkeypatch, lens_new, lens_old, hq, hkv, d, page, k, rotate, width):
    """The tcgen05 product with the rotary kernel's job in its epilogue: bit for bit what the same product followed by
    the rotary kernel (paired order) leaves in the queries and in the pages, and nothing anywhere else in the pages."""
    from prefixserve_b200 import ops
    from prefixserve_b200.ops import library, tensorcore
    monkeypatch.setattr(tensorcore, "TCGEN05_MIN_TILES", 1)
    monkeypatch.setattr(tensorcore, "TCGEN05_MIN_ROWS", 1)
    g = torch.Generator().manual_seed(sum(lens_new) + d)
    table, _, num_pages = _paged_setup(torch.bfloat16, lens_new, lens_old, hq, hkv, d, page, seed=5)
    positions = torch.cat([torch.arange(o, o + n) for o, n in zip(lens_old, lens_new)]).to(torch.int32).to(DEV)
    token_item = torch.cat([torch.full((n,), i) for i, n in enumerate(lens_new)]).to(torch.int32).to(DEV)
    t = sum(lens_new)
    h = torch.randn(t, k, generator=g).to(DEV) * 2
    pending = torch.randn(t, k, generator=g).to(torch.bfloat16).to(DEV)
    gain = (1.0 + 0.2 * torch.randn(k, generator=g)).to(DEV)
    w = (torch.randn((hq + 2 * hkv) * d, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).to(DEV)
    angles = torch.outer(torch.arange(400).float(), 1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d)))
    cos, sin = (angles.cos().to(DEV).contiguous(), angles.sin().to(DEV).contiguous()) if rotate else (None, None)
    args = dict(num_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page)
    tab = table.to(DEV)
    x = ops.NormedRows(h.clone(), pending, gain, 1e-5, torch.bfloat16)
    kv_two = torch.full((num_pages, 2, hkv, page, d), 7.0, dtype=torch.bfloat16, device=DEV)
    q_two = ops.rope_append(tensorcore.gemm_tcgen05(x.tensor(), w), positions, token_item, cos, sin, tab, kv_two, write_kv=True,
                            paired=True, **args)
    y = ops.NormedRows(h.clone(), pending, gain, 1e-5, torch.bfloat16)
    kv_one = torch.full_like(kv_two, 7.0)
    try:
        library.check(library.lib().psb_gemm_tcgen05_tile_width(width), "tile width")
        q_one = ops.qkv_rope_append(y, w, positions, token_item, cos, sin, tab, kv_one, **args)
    finally:
        library.check(library.lib().psb_gemm_tcgen05_tile_width(0), "tile width")
    assert q_one is not None and q_one.shape == (t, hq, d)
    assert torch.equal(q_one, q_two) and torch.equal(kv_one, kv_two)
    assert torch.equal(y.residual(), x.residual())
    assert library.tcgen05_status() == 0


def test_normed_rows_nobody_consumed_still_update_the_stream():
    from prefixserve_b200 import ops
    h = torch.randn(4, 64, device=DEV)
    pending = torch.randn(4, 64, device=DEV).to(torch.bfloat16)
    x = ops.NormedRows(h.clone(), pending, torch.ones(64, device=DEV), 1e-5, torch.bfloat16)
    assert torch.allclose(x.residual(), h + pending.float())
    assert torch.allclose(x.residual(), h + pending.float())  # and only once


# ---- the pair-interleaved element order, and projection + rotation + append in one kernel -----------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page", [(4, 2, 16, 16), (3, 1, 48, 8), (8, 2, 64, 16), (2, 2, 128, 32)])
def test_rope_append_in_paired_order(dtype, hq, hkv, d, page):
    from prefixserve_b200 import ops
    lens_old, lens_new = [0, 37, 5], [9, 1, 30]
    table, seqs, num_pages = _paged_setup(dtype, lens_new, lens_old, hq, hkv, d, page, seed=7)
    t = sum(lens_new)
    g = torch.Generator().manual_seed(2)
    qkv = torch.randn(t, (hq + 2 * hkv) * d, generator=g).to(dtype)
    positions = torch.cat([torch.arange(o, o + n) for o, n in zip(lens_old, lens_new)]).to(torch.int32).to(DEV)
    token_item = torch.cat([torch.full((n,), i) for i, n in enumerate(lens_new)]).to(torch.int32).to(DEV)
    angles = torch.outer(torch.arange(80).float(), 1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d)))
    cos, sin = angles.cos().to(DEV).contiguous(), angles.sin().to(DEV).contiguous()
    order = torch.tensor(ops.pair_interleaved_order(d))
    assert sorted(order.tolist()) == list(range(d))
    # the same projection output with the elements of every query and key head reordered
    heads = qkv.view(t, hq + 2 * hkv, d).clone()
    heads[:, : hq + hkv] = heads[:, : hq + hkv][:, :, order]
    results = []
    for data, paired in ((qkv, False), (heads.reshape(t, -1).contiguous(), True)):
        kv = torch.zeros(num_pages, 2, hkv, page, d, dtype=dtype, device=DEV)
        q = ops.rope_append(data.to(DEV), positions, token_item, cos, sin, table.to(DEV), kv, num_heads=hq, num_kv_heads=hkv,
                            head_dim=d, page_size=page, write_kv=True, paired=paired)
        results.append((q.cpu(), kv.cpu()))
    (q_nat, kv_nat), (q_par, kv_par) = results
    assert torch.equal(q_par, q_nat[:, :, order])
    assert torch.equal(kv_par[:, 0], kv_nat[:, 0][..., order]) and torch.equal(kv_par[:, 1], kv_nat[:, 1])


@pytest.mark.parametrize("m", [1, 5, 8, 13, 16])
@pytest.mark.parametrize("hq,hkv,d,page,k", [(8, 2, 64, 16, 512), (3, 1, 48, 8, 96), (4, 4, 128, 32, 2048), (32, 8, 64, 16, 2048),
                                              (32, 8, 128, 16, 4096), (6, 2, 128, 16, 3072)])
@pytest.mark.parametrize("rotate", [True, False])
def test_projection_rotation_and_append_in_one_kernel(m, hq, hkv, d, page, k, rotate):
    """Bit for bit what the norm-folded projection followed by the rotary kernel (paired order) produces."""
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(m + d)
    lens_old = [int(x) for x in torch.randint(0, 60, (m,), generator=g)]
    table, _, num_pages = _paged_setup(torch.bfloat16, [1] * m, lens_old, hq, hkv, d, page, seed=11)
    positions = torch.tensor(lens_old, dtype=torch.int32, device=DEV)
    token_item = torch.arange(m, dtype=torch.int32, device=DEV)
    h = torch.randn(m, k, generator=g).to(DEV) * 2
    pending = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    gain = (1.0 + 0.2 * torch.randn(k, generator=g)).to(DEV)
    w = (torch.randn((hq + 2 * hkv) * d, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).to(DEV)
    angles = torch.outer(torch.arange(80).float(), 1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d)))
    cos, sin = (angles.cos().to(DEV).contiguous(), angles.sin().to(DEV).contiguous()) if rotate else (None, None)
    args = dict(num_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page)
    x = ops.NormedRows(h.clone(), pending, gain, 1e-5, torch.bfloat16)
    kv_two = torch.zeros(num_pages, 2, hkv, page, d, dtype=torch.bfloat16, device=DEV)
    q_two = ops.rope_append(ops.linear(x, w), positions, token_item, cos, sin, table.to(DEV), kv_two, write_kv=True, paired=True, **args)
    y = ops.NormedRows(h.clone(), pending, gain, 1e-5, torch.bfloat16)
    kv_one = torch.zeros_like(kv_two)
    q_one = ops.qkv_rope_append(y, w, positions, token_item, cos, sin, table.to(DEV), kv_one, **args)
    assert q_one is not None
    assert torch.equal(q_one, q_two) and torch.equal(kv_one, kv_two)
    assert torch.equal(y.residual(), x.residual())
    assert float(kv_one.float().abs().sum()) > 0


# ---- the tcgen05 / TMEM / TMA product for many rows -----------------------------------------------------------------

@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (17, 40, 8), (130, 333, 264), (2048, 3072, 2048), (300, 2048, 8192),
                                   (1000, 1000, 1000), (129, 128256 // 16, 96)])
def test_gemm_tcgen05(m, n, k):
    from prefixserve_b200.ops import library
    from prefixserve_b200.ops.tensorcore import gemm_tcgen05
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = torch.randn(n, k, device=DEV).to(torch.bfloat16)
    got = gemm_tcgen05(x, w)
    assert library.tcgen05_status() == 0, "a bounded wait in the kernel gave up"
    want = x.double() @ w.double().t()
    assert got.shape == (m, n) and got.dtype == torch.bfloat16
    assert torch.allclose(got.double(), want, rtol=1e-2, atol=1e-2 * math.sqrt(k)), float((got.double() - want).abs().max())
    # the same rows inside another batch give the same bits (tile-local sums, fixed k order)
    if m >= 130:
        part = gemm_tcgen05(x[:129].contiguous(), w)
        assert torch.equal(part, got[:129])


@pytest.mark.parametrize("m,n,k", [(128, 192, 64), (130, 333, 264), (2048, 3072, 2048), (700, 2000, 1000), (129, 8016, 96)])
def test_gemm_tcgen05_tile_widths_agree(m, n, k):
    """The launcher picks output tiles of 256, 240, 192 or 128 columns by how they fill the SMs; a sum does not depend on it."""
    from prefixserve_b200.ops import library
    from prefixserve_b200.ops.tensorcore import gemm_tcgen05
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = torch.randn(n, k, device=DEV).to(torch.bfloat16)
    got = {}
    try:
        for width in (128, 192, 240, 256):
            library.check(library.lib().psb_gemm_tcgen05_tile_width(width), "tile width")
            got[width] = gemm_tcgen05(x, w)
    finally:
        library.check(library.lib().psb_gemm_tcgen05_tile_width(0), "tile width")
    assert library.tcgen05_status() == 0
    assert torch.equal(got[192], got[256]) and torch.equal(got[128], got[256]) and torch.equal(got[240], got[256])
    want = x.double() @ w.double().t()
    assert torch.allclose(got[192].double(), want, rtol=1e-2, atol=1e-2 * math.sqrt(k))


@pytest.mark.parametrize("width", [0, 128, 256])
@pytest.mark.parametrize("m,inter,k", [(128, 128, 64), (50, 40, 24), (257, 333, 264), (2048, 8192, 2048), (512, 1000, 2048)])
def test_gemm_tcgen05_gated(m, inter, k, width):
    from prefixserve_b200.ops import library
    from prefixserve_b200.ops.tensorcore import gemm_tcgen05_gated
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, device=DEV) / math.sqrt(k)).to(torch.bfloat16)
    try:
        library.check(library.lib().psb_gemm_tcgen05_tile_width(width), "tile width")
        got = gemm_tcgen05_gated(x, w)
    finally:
        library.check(library.lib().psb_gemm_tcgen05_tile_width(0), "tile width")
    assert library.tcgen05_status() == 0
    y = (x.double() @ w.double().t()).to(torch.bfloat16).double()  # the reference rounds the projections first
    want = torch.nn.functional.silu(y[:, :inter]) * y[:, inter:]
    assert got.shape == (m, inter)
    assert torch.allclose(got.double(), want, rtol=3e-2, atol=3e-2), float((got.double() - want).abs().max())


# ---- the product for a few dozen rows: rows in the instruction's N dimension, the contraction shared out over a cluster --

@pytest.fixture
def fewrows_splits():
    from prefixserve_b200.ops import library
    def force(n):
        library.check(library.lib().psb_gemm_fewrows_splits(n), "splits")
    yield force
    force(0)


@pytest.mark.parametrize("splits", [0, 1, 4, 8])
@pytest.mark.parametrize("m,n,k", [(17, 256, 512), (64, 2048, 2048), (33, 333, 264), (40, 3072, 2048), (64, 2048, 8192),
                                   (50, 1000, 1000), (20, 128, 64), (31, 8016, 96)])
def test_gemm_fewrows(m, n, k, splits, fewrows_splits):
    from prefixserve_b200.ops import library
    from prefixserve_b200.ops.tensorcore import gemm_fewrows
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = torch.randn(n, k, device=DEV).to(torch.bfloat16)
    fewrows_splits(splits)
    got = gemm_fewrows(x, w)
    assert library.tcgen05_status() == 0, "a bounded wait in the kernel gave up"
    want = x.double() @ w.double().t()
    assert got.shape == (m, n) and got.dtype == torch.bfloat16
    assert torch.allclose(got.double(), want, rtol=1e-2, atol=1e-2 * math.sqrt(k)), float((got.double() - want).abs().max())
    # the same rows inside another batch give the same bits (a token's sums do not depend on its neighbours)
    part = gemm_fewrows(x[:17].contiguous(), w)
    assert torch.equal(part, got[:17])
    assert torch.equal(gemm_fewrows(x, w), got)


@pytest.mark.parametrize("splits", [0, 2, 8])
@pytest.mark.parametrize("m,inter,k", [(64, 8192, 2048), (50, 40, 128), (17, 333, 264), (33, 1000, 2048)])
def test_gemm_fewrows_gated(m, inter, k, splits, fewrows_splits):
    from prefixserve_b200.ops import library
    from prefixserve_b200.ops.tensorcore import gemm_fewrows_gated
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, device=DEV) / math.sqrt(k)).to(torch.bfloat16)
    fewrows_splits(splits)
    y = (x.double() @ w.double().t()).to(torch.bfloat16).double()  # the reference rounds the projections first
    for name, code, f in (("silu", 0, torch.nn.functional.silu),
                          ("gelu_tanh", 1, lambda v: torch.nn.functional.gelu(v, approximate="tanh"))):
        got = gemm_fewrows_gated(x, w, code)
        assert library.tcgen05_status() == 0
        want = f(y[:, :inter]) * y[:, inter:]
        assert got.shape == (m, inter)
        assert torch.allclose(got.double(), want, rtol=3e-2, atol=3e-2), (name, float((got.double() - want).abs().max()))


@pytest.mark.parametrize("m", [17, 33, 64])
@pytest.mark.parametrize("hq,hkv,d,page,k", [(8, 2, 64, 16, 512), (3, 1, 48, 8, 96), (4, 4, 128, 32, 2048), (32, 8, 64, 16, 2048),
                                              (6, 2, 128, 16, 3072)])
@pytest.mark.parametrize("rotate", [True, False])
def test_fewrows_projection_rotation_and_append_in_one_kernel(m, hq, hkv, d, page, k, rotate, monkeypatch):
    """Bit for bit what the same product followed by the rotary kernel (paired order) produces, for single tokens of
    many requests and for one portion."""
    from prefixserve_b200 import ops
    from prefixserve_b200.ops import library, tensorcore
    monkeypatch.setattr(tensorcore, "FEWROWS_MAX", {"plain": 64, "gated": 64, "rope": 64})
    g = torch.Generator().manual_seed(m + d)
    for portion in (False, True):
        if portion:
            lens_old, lens_new = [23], [m]
        else:
            lens_old, lens_new = [int(x) for x in torch.randint(0, 60, (m,), generator=g)], [1] * m
        table, _, num_pages = _paged_setup(torch.bfloat16, lens_new, lens_old, hq, hkv, d, page, seed=11)
        positions = torch.cat([torch.arange(o, o + n) for o, n in zip(lens_old, lens_new)]).to(torch.int32).to(DEV)
        token_item = torch.cat([torch.full((n,), i) for i, n in enumerate(lens_new)]).to(torch.int32).to(DEV)
        h = torch.randn(m, k, generator=g).to(DEV) * 2
        pending = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
        gain = (1.0 + 0.2 * torch.randn(k, generator=g)).to(DEV)
        w = (torch.randn((hq + 2 * hkv) * d, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).to(DEV)
        angles = torch.outer(torch.arange(120).float(), 1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d)))
        cos, sin = (angles.cos().to(DEV).contiguous(), angles.sin().to(DEV).contiguous()) if rotate else (None, None)
        args = dict(num_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page)
        x = ops.NormedRows(h.clone(), pending, gain, 1e-5, torch.bfloat16)
        kv_two = torch.zeros(num_pages, 2, hkv, page, d, dtype=torch.bfloat16, device=DEV)
        q_two = ops.rope_append(ops.linear(x, w), positions, token_item, cos, sin, table.to(DEV), kv_two, write_kv=True, paired=True, **args)
        y = ops.NormedRows(h.clone(), pending, gain, 1e-5, torch.bfloat16)
        kv_one = torch.zeros_like(kv_two)
        before = library.launch_counts["gemm_fewrows_rope"]
        q_one = ops.qkv_rope_append(y, w, positions, token_item, cos, sin, table.to(DEV), kv_one, **args)
        assert q_one is not None and library.launch_counts["gemm_fewrows_rope"] == before + 1
        assert library.tcgen05_status() == 0
        assert torch.equal(q_one, q_two) and torch.equal(kv_one, kv_two)
        assert float(kv_one.float().abs().sum()) > 0
        # and against plain arithmetic on the normalised rows
        xn = x.tensor().double()
        want_v = (xn @ w.double().t())[:, (hq + hkv) * d:].to(torch.bfloat16)
        for tok in (0, m - 1):
            pos = int(positions[tok])
            pg = int(table[int(token_item[tok]), pos // page])
            got_v = kv_one[pg, 1, :, pos % page].reshape(-1)
            assert torch.allclose(got_v.double(), want_v[tok].double(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("splits", [0, 1, 4])
@pytest.mark.parametrize("m,hidden,inter", [(17, 256, 384), (32, 2048, 8192), (24, 200, 328), (9, 2048, 1000)])
def test_fewrows_products_around_a_norm(m, hidden, inter, splits, fewrows_splits, monkeypatch):
    """The product in front of a norm adds itself to the stream and leaves the gained rows and the shares of the sums
    of squares; the products behind it (plain, gated) scale their sums.  Against float64, and against the same chain
    through the norm's own kernel."""
    from prefixserve_b200 import ops
    from prefixserve_b200.ops import library, tensorcore
    monkeypatch.setattr(tensorcore, "FEWROWS_MAX", {"plain": 64, "gated": 64, "rope": 64})
    fewrows_splits(splits)
    eps = 1e-5
    g = torch.Generator().manual_seed(m + hidden)
    a = torch.randn(m, inter, generator=g).to(torch.bfloat16).to(DEV)
    w_front = (torch.randn(hidden, inter, generator=g) / math.sqrt(inter)).to(torch.bfloat16).to(DEV)
    h = (torch.randn(m, hidden, generator=g) * 2).to(DEV)
    gain = (1.0 + 0.2 * torch.randn(hidden, generator=g)).to(DEV)
    w_plain = (torch.randn(333, hidden, generator=g) / math.sqrt(hidden)).to(torch.bfloat16).to(DEV)
    w_gated = (torch.randn(2 * 200, hidden, generator=g) / math.sqrt(hidden)).to(torch.bfloat16).to(DEV)
    # float64: the product rounded to bfloat16, the residual sum, the norm, the products behind it
    delta = (a.double() @ w_front.double().t()).to(torch.bfloat16).double()
    v = h.double() + delta
    normed = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * gain.double()
    want_plain = normed @ w_plain.double().t()
    y = (normed @ w_gated.double().t()).to(torch.bfloat16).double()
    want_gated = torch.nn.functional.silu(y[:, :200]) * y[:, 200:]
    for kind, w_behind, want in (("plain", w_plain, want_plain), ("gated", w_gated, want_gated)):
        stream = h.clone()
        x = ops.NormedRows(stream, ops.PendingProduct(a, w_front), gain, eps, torch.bfloat16)
        before = library.launch_counts.copy()
        got = ops.linear(x, w_behind) if kind == "plain" else ops.gated_linear(x, w_behind)
        ran = library.launch_counts - before
        assert ran["gemm_fewrows_add_norm"] == 1 and ran["add_rmsnorm"] == 0, ran
        assert library.tcgen05_status() == 0
        # the stream after the sum (the product is rounded to bfloat16 on its way in: a unit in its last place may differ from float64's)
        assert torch.allclose(x.residual().double(), v, rtol=0, atol=2.0 ** -8 * float(delta.abs().max())), kind
        tol = 3e-2 * float(want.abs().max())
        assert float((got.double() - want).abs().max()) <= tol, (kind, float((got.double() - want).abs().max()), tol)
        # the same through the norm's own kernel: no further from float64 than a factor
        stream2 = h.clone()
        y2 = ops.NormedRows(stream2, ops.linear(a, w_front), gain, eps, torch.bfloat16)
        unfused = ops.linear(y2.tensor(), w_behind) if kind == "plain" else ops.gated_linear(y2.tensor(), w_behind)
        err, err2 = float((got.double() - want).abs().max()), float((unfused.double() - want).abs().max())
        assert err <= 2.0 * err2 + 1e-3 * float(want.abs().max()), (kind, err, err2)
        assert torch.equal(stream, stream2)   # the same float32 stream bit for bit


def test_a_bounded_wait_that_runs_out_gives_up_and_says_so():
    """The tensor-core kernels wait on mbarriers through one bounded primitive.  Its give-up path runs here on a
    barrier that nobody arrives at, with a limit of a few hundred polls, in a kernel of one warp that has nothing in
    flight: the wait returns false, raises the abort flag and leaves its caller's code in the status word, which the
    host reads and finds cleared afterwards.  The product kernels' own status words stay untouched."""
    from prefixserve_b200.ops import library
    assert library.tcgen05_status() == 0
    out = torch.full((3,), -1, dtype=torch.int32, device=DEV)
    for limit, who in ((256, 7), (1000, 42)):
        library.check(library.lib().psb_selftest_bounded_wait(limit, who, out.data_ptr(), library.stream_handle()), "selftest")
        assert out.tolist() == [0, 1, who]
    assert library.tcgen05_status() == 0                       # not the product kernels' word
    assert library.lib().psb_selftest_bounded_wait(1 << 20, 1, out.data_ptr(), None) != 0   # long waits are refused
