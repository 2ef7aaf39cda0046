"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

Some embedders cannot call cudaMalloc around a decode step: a host process with a fixed device-memory budget, code
running inside another component's stream capture, C callers without a caching allocator.  For them the library keeps
the split-KV scratch in a fixed 4 MiB array of its own.  This test drives that entry point with ctypes exactly as a C
caller would, twice in a row on different inputs (the array keeps the previous call's contents), and compares with the
entry point that takes a caller-provided scratch buffer and with a float32 attention written in plain torch over the
pages gathered by the table (the two entry points share their kernels, so agreement between them alone would let a
fault of both pass).  It also checks that a request beyond the fixed size is refused without launching.

The file name makes pytest collect it last, so a failure here cannot hide the result of any other test.
"""

import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
MAX_FLOATS = 1 << 20


def _library():
    from prefixserve_b200.build import ensure_kernels
    lib = ctypes.CDLL(str(ensure_kernels()))
    P, I, F = c_void_p, c_int, c_float
    lib.psb_attention_decode_bf16.argtypes = [P, P, P, I, P, P, P, P, P, I, I, I, I, I, I, F, I, I, I, P]
    lib.psb_attention_decode_bf16.restype = c_int
    lib.psb_attention_decode_bf16_static.argtypes = [P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, I, I, P]
    lib.psb_attention_decode_bf16_static.restype = c_int
    lib.psb_last_error.restype = ctypes.c_char_p
    return lib


def _problem(seed, kv_lens, hq=8, hkv=2, d=64, page=16):
    g = torch.Generator().manual_seed(seed)
    b = len(kv_lens)
    pages_per = -(-max(kv_lens) // page)
    num_pages = b * pages_per + 3
    kv = torch.randn(num_pages, 2, hkv, page, d, generator=g).to(torch.bfloat16).to(DEV)
    table = torch.randperm(num_pages, generator=g)[: b * pages_per].to(torch.int32).view(b, pages_per).contiguous().to(DEV)
    q = torch.randn(b, hq, d, generator=g).to(torch.bfloat16).to(DEV)
    item_start = torch.arange(b + 1, dtype=torch.int32, device=DEV)
    kv_len = torch.tensor(kv_lens, dtype=torch.int32, device=DEV)
    return dict(q=q, kv=kv, table=table, item_start=item_start, kv_len=kv_len, b=b, hq=hq, hkv=hkv, d=d, page=page,
                width=pages_per)


def _run(lib, pr, chunk, static):
    max_splits = -(-int(pr["kv_len"].max()) // chunk)
    out = torch.zeros(pr["b"], pr["hq"] * pr["d"], dtype=torch.bfloat16, device=DEV)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    scale = 1.0 / pr["d"] ** 0.5
    common_tail = (pr["b"], pr["hq"], pr["hkv"], pr["d"], pr["page"], 0, scale, chunk, max_splits, 1, stream)
    head = (pr["q"].data_ptr(), pr["kv"].data_ptr(), pr["table"].data_ptr(), pr["width"], pr["item_start"].data_ptr(),
            pr["kv_len"].data_ptr(), out.data_ptr())
    if static:
        rc = lib.psb_attention_decode_bf16_static(*head, *common_tail)
    else:
        n = pr["b"] * pr["hq"] * max_splits
        part_o = torch.empty(n * pr["d"], dtype=torch.float32, device=DEV)
        part_ml = torch.empty(n * 2, dtype=torch.float32, device=DEV)
        rc = lib.psb_attention_decode_bf16(*head, part_o.data_ptr(), part_ml.data_ptr(), *common_tail)
    assert rc == 0, lib.psb_last_error().decode()
    torch.cuda.synchronize()
    return out


def _plain_attention(pr):
    """softmax(q k^T / sqrt(D)) v per request in float32, keys and values gathered page by page through the table."""
    b, hq, hkv, d, page = pr["b"], pr["hq"], pr["hkv"], pr["d"], pr["page"]
    kv, table, q = pr["kv"].float().cpu(), pr["table"].cpu(), pr["q"].float().cpu()
    out = torch.empty(b, hq * d)
    for i, n in enumerate(pr["kv_len"].tolist()):
        pages = kv[table[i].long()]                                            # [pages, 2, hkv, page, D]
        keys = pages[:, 0].permute(0, 2, 1, 3).reshape(-1, hkv, d)[:n]           # [n, hkv, D] in position order
        vals = pages[:, 1].permute(0, 2, 1, 3).reshape(-1, hkv, d)[:n]
        keys, vals = keys.repeat_interleave(hq // hkv, dim=1), vals.repeat_interleave(hq // hkv, dim=1)
        probs = torch.softmax(torch.einsum("hd,nhd->hn", q[i], keys) / d ** 0.5, dim=-1)
        out[i] = torch.einsum("hn,nhd->hd", probs, vals).reshape(hq * d)
    return out


def test_static_scratch_entry_point_matches_the_allocating_one_twice_in_a_row():
    lib = _library()
    # two different problems back to back: the second call finds the first call's partial results in the array
    for seed, kv_lens, chunk in ((1, [700, 33, 1, 256], 64), (2, [90, 1300, 64], 128)):
        pr = _problem(seed, kv_lens)
        want = _run(lib, pr, chunk, static=False)
        got = _run(lib, pr, chunk, static=True)
        assert torch.isfinite(got.float()).all()
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        plain = _plain_attention(pr)
        assert torch.allclose(got.float().cpu(), plain, atol=2e-2, rtol=2e-2), float((got.float().cpu() - plain).abs().max())
        assert torch.allclose(want.float().cpu(), plain, atol=2e-2, rtol=2e-2)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = _library()
    pr = _problem(3, [64] * 4, hq=32, hkv=8)
    out = torch.zeros(4, 32 * 64, dtype=torch.bfloat16, device=DEV)
    too_many = MAX_FLOATS // (4 * 32 * 66) + 1
    rc = lib.psb_attention_decode_bf16_static(
        pr["q"].data_ptr(), pr["kv"].data_ptr(), pr["table"].data_ptr(), pr["width"], pr["item_start"].data_ptr(),
        pr["kv_len"].data_ptr(), out.data_ptr(), 4, 32, 8, 64, 16, 0, 0.125, 64, too_many, 1,
        c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0 and b"exceed the built-in scratch" in lib.psb_last_error()
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0  # nothing was launched
