"""Host-side faces of the kernels: argument checks, output allocation, launch.

Tensors are handed to the C ABI as raw device pointers on the current CUDA
stream.  Everything here refuses CPU tensors: there is no CPU path.
"""

from __future__ import annotations

import math

import torch

from .deferred import NormedRows, PendingProduct
from .library import KernelError, check, lib, stream_handle

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not one of float32, bfloat16") from None


def _dev(t: torch.Tensor, what: str) -> torch.Tensor:
    if not t.is_cuda:
        raise KernelError(f"{what} is on {t.device}; the kernels run on a CUDA device only")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous, strides are {t.stride()}")
    return t


def _i32(t: torch.Tensor, what: str) -> torch.Tensor:
    if t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, is {t.dtype}")
    return _dev(t, what)


def _stream() -> int:
    return stream_handle()


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """h[t] = float32(table[ids[t]])."""
    _i32(ids, "token ids")
    _dev(table, "embedding table")
    t, (v, h) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((t, h), dtype=torch.float32, device=ids.device)
    check(lib().psb_embedding(ids.data_ptr(), table.data_ptr(), _code(table, "embedding table"), out.data_ptr(),
                              t, h, v, _stream()), "embedding")
    return out


def add_rmsnorm(h: torch.Tensor, delta: torch.Tensor | None, gain: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: torch.Tensor | None = None) -> torch.Tensor:
    """h += delta (float32, in place, unless ``rows``); returns gain * rmsnorm(h) for all or the chosen rows."""
    if isinstance(delta, PendingProduct):
        delta = delta.tensor()
    _dev(h, "residual stream")
    if h.dtype != torch.float32 or h.dim() != 2:
        raise KernelError(f"residual stream must be float32 [T, H], is {h.dtype} {tuple(h.shape)}")
    width = h.shape[1]
    if gain.dtype != torch.float32 or gain.numel() != width:
        raise KernelError(f"norm gain must be float32 [{width}], is {gain.dtype} {tuple(gain.shape)}")
    _dev(gain, "norm gain")
    dcode = F32
    if delta is not None:
        _dev(delta, "sublayer output")
        if delta.shape != h.shape:
            raise KernelError(f"sublayer output {tuple(delta.shape)} does not match the stream {tuple(h.shape)}")
        dcode = _code(delta, "sublayer output")
    n = h.shape[0]
    if rows is not None:
        _i32(rows, "row index")
        n = rows.numel()
    x = torch.empty((n, width), dtype=out_dtype, device=h.device)
    check(lib().psb_add_rmsnorm(h.data_ptr(), _ptr(delta), dcode, gain.data_ptr(), _ptr(rows), x.data_ptr(),
                                _code(x, "norm output"), n, width, float(eps), 0 if rows is not None else 1, _stream()),
          "add_rmsnorm")
    return x


def gemm_nt_simt(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, out: torch.Tensor | None = None,
                 accumulate: bool = False) -> torch.Tensor:
    """a[M,K] @ w[N,K]^T with float32 multiply-adds on the CUDA cores."""
    _dev(a, "left operand")
    _dev(w, "weight")
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1]:
        raise KernelError(f"cannot multiply {tuple(a.shape)} by the transpose of {tuple(w.shape)}")
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    check(lib().psb_gemm_nt(a.data_ptr(), _code(a, "left operand"), w.data_ptr(), _code(w, "weight"), out.data_ptr(),
                            _code(out, "product"), m, n, k, k, k, n, 1 if accumulate else 0, _stream()), "gemm_nt")
    return out


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """x[M,K] @ w[N,K]^T, accumulated in float32.

    bfloat16 x bfloat16 goes to the tensor-core path; every other mix (all of
    the 32-bit path, and weights a checkpoint stores in float32) goes to the
    float32 CUDA-core kernel, so that path never touches a reduced-precision
    matrix mode.
    """
    if isinstance(x, NormedRows):
        if x.fusable and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
            from .tensorcore import norm_linear_bf16
            y = norm_linear_bf16(x, w, out_dtype or x.dtype)
            if y is not None:
                return y
        if (out_dtype or x.dtype) == torch.bfloat16 and w.dtype == torch.bfloat16:
            from .tensorcore import fewrows_behind_norm
            y = fewrows_behind_norm(x, w, "plain")
            if y is not None:
                return y
        x = x.tensor()
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        from .tensorcore import linear_bf16
        return linear_bf16(x, w, out_dtype)
    return gemm_nt_simt(x, w, out_dtype)


def last_product(x: torch.Tensor, w: torch.Tensor, ctx=None):
    """A sublayer's last product, x @ w^T, whose only reader is the residual sum in front of the next norm.  Where the
    step says that every norm downstream takes one (``ctx.extras["lazy_products"]``) and the rows are few enough for
    the kernel that can carry that sum and the norm's share in its epilogue, the product is handed on unrun
    (``PendingProduct``); otherwise it runs now."""
    extras = getattr(ctx, "extras", None)
    if extras is not None and extras.get("lazy_products") and x.dim() == 2 and x.is_cuda:
        from .tensorcore import fewrows_lazy_ok
        if fewrows_lazy_ok(x, w):
            return PendingProduct(x, w)
    return linear(x, w)


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}  # the codes the kernels know (PsbAct in common.cuh)


def activation_code(name: str) -> int:
    try:
        return ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"activation {name!r} is not built (one of {sorted(ACTIVATIONS)})") from None


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    """act(x Wg^T) * (x Wu^T) for W = [gate rows; up rows]: fused for bfloat16 rows, else product then activation."""
    code = activation_code(activation)
    if isinstance(x, NormedRows):
        if x.fusable and x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16:
            from .tensorcore import norm_gated_linear_bf16
            act = norm_gated_linear_bf16(x, w_gate_up, code)
            if act is not None:
                return act
        if w_gate_up.dtype == torch.bfloat16:
            from .tensorcore import fewrows_behind_norm
            act = fewrows_behind_norm(x, w_gate_up, "gated", activation=code)
            if act is not None:
                return act
        x = x.tensor()
    if x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16:
        from .tensorcore import gated_linear_bf16
        _dev(x, "left operand"), _dev(w_gate_up, "weight")
        act = gated_linear_bf16(x, w_gate_up, activation=code)
        if act is not None:
            return act
    return act_mul(linear(x, w_gate_up), activation)


def rope_append(qkv: torch.Tensor, positions: torch.Tensor, token_item: torch.Tensor, cos: torch.Tensor | None,
                sin: torch.Tensor | None, table: torch.Tensor | None, kv: torch.Tensor | None, *, num_heads: int,
                num_kv_heads: int, head_dim: int, page_size: int, write_kv: bool, paired: bool = False,
                rotary_dim: int | None = None, interleaved: bool = False) -> torch.Tensor:
    """Rotates queries (and keys); stores rotated keys and values in the pages. Returns q [T, hq, D].

    ``paired``: every query and key head comes (and goes) with its elements in the pair-interleaved order of
    ``pair_interleaved_order``; the rotary kernel's header says why that is harmless.
    ``rotary_dim``: only the first so many elements of a head turn (default: all; the tables then hold
    rotary_dim/2 angles); ``interleaved``: element 2j turns with 2j+1 instead of j with j + rotary_dim/2."""
    _dev(qkv, "projection output")
    t = qkv.shape[0]
    hkv_in = num_kv_heads if write_kv else 0
    want = (num_heads + 2 * hkv_in) * head_dim
    if qkv.dim() != 2 or qkv.shape[1] != want:
        raise KernelError(f"projection output must be [T, {want}], is {tuple(qkv.shape)}")
    _i32(positions, "positions")
    _i32(token_item, "token-to-item map")
    rotate = cos is not None
    max_pos = 0
    rotary_dim = head_dim if rotary_dim is None else int(rotary_dim)
    if rotary_dim < 2 or rotary_dim > head_dim or rotary_dim % 2:
        raise KernelError(f"rotary_dim {rotary_dim} must be even and within the head size {head_dim}")
    if paired and (rotary_dim != head_dim or interleaved):
        raise KernelError("the paired element order goes with the split-half rotation of a whole head only")
    if rotate:
        assert sin is not None
        _dev(cos, "cos table"), _dev(sin, "sin table")
        if cos.dtype != torch.float32 or cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] != rotary_dim // 2:
            raise KernelError(f"angle tables must be float32 [positions, {rotary_dim // 2}], are {cos.dtype} {tuple(cos.shape)}")
        max_pos = cos.shape[0]
    width = num_pages = 0
    kv_code = _code(qkv, "projection output")
    if write_kv:
        if kv is None or table is None:
            raise KernelError("appending to the cache needs the cache entry and the page table")
        _dev(kv, "cache entry"), _i32(table, "page table")
        if kv.dim() != 5 or tuple(kv.shape[1:]) != (2, num_kv_heads, page_size, head_dim):
            raise KernelError(f"cache entry must be [pages, 2, {num_kv_heads}, {page_size}, {head_dim}], is {tuple(kv.shape)}")
        num_pages, width, kv_code = kv.shape[0], table.shape[1], _code(kv, "cache entry")
    q = torch.empty((t, num_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    check(lib().psb_rope_append(qkv.data_ptr(), _code(qkv, "projection output"), positions.data_ptr(),
                                token_item.data_ptr(), _ptr(cos), _ptr(sin), _ptr(table) if write_kv else None, width,
                                _ptr(kv) if write_kv else None, kv_code, q.data_ptr(), t, num_heads, hkv_in, head_dim,
                                page_size, num_pages, max_pos, 1 if rotate else 0, 1 if write_kv else 0, 1 if paired else 0,
                                rotary_dim, 1 if interleaved else 0, _stream()),
          "rope_append")
    return q


def pair_interleaved_order(head_dim: int) -> list[int]:
    """For a head size that is a multiple of 16: natural element index for each stored index when 8 elements of the
    first half are followed by the 8 elements they are rotated with (split-half rotation pairs d with d + D/2)."""
    if head_dim % 16:
        raise KernelError(f"a head size of {head_dim} cannot be pair-interleaved (multiples of 16 only)")
    order: list[int] = []
    for block in range(head_dim // 16):
        order += list(range(8 * block, 8 * block + 8)) + list(range(head_dim // 2 + 8 * block, head_dim // 2 + 8 * block + 8))
    return order


def qkv_rope_append(x: NormedRows, w_qkv: torch.Tensor, positions: torch.Tensor, token_item: torch.Tensor,
                    cos: torch.Tensor | None, sin: torch.Tensor | None, table: torch.Tensor, kv: torch.Tensor, *,
                    num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> torch.Tensor | None:
    """rmsnorm(h + pending) @ w_qkv^T, rotation and append to the pages, for bfloat16 tokens and a projection whose
    query and key rows are pair-interleaved: one kernel for few tokens (the norm folded in as well), the norm's kernel
    and one product that rotates and stores in its epilogue for many.  Returns q [T, hq, D], or None when neither kernel
    takes the case (the caller then runs the product and ``rope_append(..., paired=True)``)."""
    from .tensorcore import norm_qkv_rope_bf16, tcgen05_qkv_rope_bf16
    if not (x.rows is None and x.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16
            and kv.dtype == torch.bfloat16 and head_dim % 16 == 0 and page_size & (page_size - 1) == 0):
        return None
    _i32(positions, "positions"), _i32(token_item, "token-to-item map"), _i32(table, "page table"), _dev(kv, "cache entry")
    if kv.dim() != 5 or tuple(kv.shape[1:]) != (2, num_kv_heads, page_size, head_dim):
        raise KernelError(f"cache entry must be [pages, 2, {num_kv_heads}, {page_size}, {head_dim}], is {tuple(kv.shape)}")
    if w_qkv.shape[0] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError(f"projection has {w_qkv.shape[0]} rows, not {(num_heads + 2 * num_kv_heads) * head_dim}")
    if cos is not None and (sin is None or cos.dtype != torch.float32 or cos.shape != sin.shape or cos.dim() != 2
                            or cos.shape[1] != head_dim // 2):
        raise KernelError(f"angle tables must be float32 [positions, {head_dim // 2}]")
    if x.fusable:
        q = norm_qkv_rope_bf16(x, w_qkv, positions, token_item, cos, sin, table, kv, num_heads, num_kv_heads, head_dim, page_size)
        if q is not None:
            return q
    from .tensorcore import fewrows_behind_norm
    q = fewrows_behind_norm(x, w_qkv, "rope", rope=(positions, token_item, cos, sin, table, kv, num_heads, num_kv_heads, head_dim, page_size))
    if q is not None:
        return q
    return tcgen05_qkv_rope_bf16(x.tensor(), w_qkv, positions, token_item, cos, sin, table, kv, num_heads, num_kv_heads,
                                 head_dim, page_size)


def attention_generic(q: torch.Tensor, kv: torch.Tensor, table: torch.Tensor, positions: torch.Tensor,
                      token_item: torch.Tensor, *, window: int | None, scale: float) -> torch.Tensor:
    _dev(q, "queries"), _dev(kv, "cache entry")
    _i32(table, "page table"), _i32(positions, "positions"), _i32(token_item, "token-to-item map")
    t, hq, d = q.shape
    _, two, hkv, page, dk = kv.shape
    if two != 2 or dk != d:
        raise KernelError(f"cache entry {tuple(kv.shape)} does not fit queries {tuple(q.shape)}")
    out = torch.empty((t, hq * d), dtype=q.dtype, device=q.device)
    check(lib().psb_attention_generic(q.data_ptr(), _code(q, "queries"), kv.data_ptr(), _code(kv, "cache entry"),
                                      table.data_ptr(), table.shape[1], positions.data_ptr(), token_item.data_ptr(),
                                      out.data_ptr(), t, hq, hkv, d, page, int(window or 0), float(scale), _stream()),
          "attention")
    return out


def attention(q: torch.Tensor, kv: torch.Tensor, table: torch.Tensor, positions: torch.Tensor,
              token_item: torch.Tensor, *, window: int | None = None, scale: float | None = None,
              ctx=None) -> torch.Tensor:
    """Causal grouped-query attention of the step's tokens over their requests' pages -> [T, hq*D]."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and ctx is not None:
        from .tensorcore import attention_bf16
        _dev(q, "queries"), _dev(kv, "cache entry"), _i32(table, "page table")
        if q.shape[1] % kv.shape[2] or kv.shape[4] != q.shape[2] or kv.shape[1] != 2:
            raise KernelError(f"cache entry {tuple(kv.shape)} does not fit queries {tuple(q.shape)}")
        extras = getattr(ctx, "extras", None)
        fast = attention_bf16(q, kv, table, ctx.item_start, ctx.kv_len, None, None, window=window, scale=scale,
                              static_kv_len=extras.get("static_kv_len") if extras is not None else None,
                              plans=extras, items=ctx.items, token_item=_i32(token_item, "token-to-item map"))
        if fast is not None:
            return fast
    return attention_generic(q, kv, table, positions, token_item, window=window, scale=scale)


def act_mul(gate_up: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    """[T, 2I] -> act(first half) * second half, [T, I]."""
    _dev(gate_up, "gate/up projection")
    t, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError(f"gate/up projection must have an even width, has {two_i}")
    out = torch.empty((t, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    check(lib().psb_silu_mul(gate_up.data_ptr(), _code(gate_up, "gate/up projection"), out.data_ptr(), t, two_i // 2,
                             activation_code(activation), _stream()), "silu_mul")
    return out


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """[T, 2I] -> silu(first half) * second half, [T, I]."""
    return act_mul(gate_up, "silu")


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """h += delta in place (h float32, delta float32 or bfloat16 of the same shape); returns h."""
    if isinstance(delta, PendingProduct):
        delta = delta.tensor()
    _dev(h, "residual stream"), _dev(delta, "sublayer output")
    if h.dtype != torch.float32 or delta.shape != h.shape:
        raise KernelError(f"residual stream must be float32 and the output must match it: {h.dtype} {tuple(h.shape)} vs {tuple(delta.shape)}")
    check(lib().psb_residual_add(h.data_ptr(), delta.data_ptr(), _code(delta, "sublayer output"), h.numel(), _stream()), "residual_add")
    return h


def sample(logits: torch.Tensor, temperature: torch.Tensor | None = None, seed: torch.Tensor | None = None,
           position: torch.Tensor | None = None) -> torch.Tensor:
    """Arg max (temperature absent or 0) or Gumbel-max sampling per row -> int32 [S]."""
    _dev(logits, "logits")
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise KernelError(f"logits must be float32 [S, V], are {logits.dtype} {tuple(logits.shape)}")
    s, v = logits.shape
    if temperature is not None:
        if seed is None or position is None:
            raise KernelError("temperature sampling needs seed and position per row")
        _dev(temperature, "temperature"), _dev(seed, "seed"), _i32(position, "position")
        if temperature.dtype != torch.float32 or seed.dtype != torch.int64:
            raise KernelError("temperature must be float32 and seed int64")
        if temperature.numel() != s or seed.numel() != s or position.numel() != s:
            raise KernelError("temperature, seed and position need one entry per logits row")
    out = torch.empty((s,), dtype=torch.int32, device=logits.device)
    need = lib().psb_sample_scratch_bytes(s, v)
    scratch = torch.empty((need,), dtype=torch.uint8, device=logits.device) if need else None
    check(lib().psb_sample(logits.data_ptr(), _ptr(temperature), _ptr(seed), _ptr(position), out.data_ptr(),
                           _ptr(scratch), s, v, _stream()), "sample")
    return out


def sample_slots(logits: torch.Tensor, records: torch.Tensor, row_slot: torch.Tensor) -> torch.Tensor:
    """The same choice with each row's temperature, seed and position read on the device from the record of the row's
    request slot (``records`` int32 [num_slots, words]: position, temperature bits, seed low, seed high) -> int32 [S]."""
    _dev(logits, "logits"), _i32(records, "slot records"), _i32(row_slot, "slot of each row")
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise KernelError(f"logits must be float32 [S, V], are {logits.dtype} {tuple(logits.shape)}")
    s, v = logits.shape
    if records.dim() != 2 or records.shape[1] < 4 or row_slot.numel() != s:
        raise KernelError(f"slot records must be [slots, >=4] and one slot per logits row is needed, got {tuple(records.shape)}, "
                          f"{row_slot.numel()} slots for {s} rows")
    out = torch.empty((s,), dtype=torch.int32, device=logits.device)
    need = lib().psb_sample_scratch_bytes(s, v)
    scratch = torch.empty((need,), dtype=torch.uint8, device=logits.device) if need else None
    check(lib().psb_sample_slots(logits.data_ptr(), records.data_ptr(), row_slot.data_ptr(), records.shape[1], out.data_ptr(),
                                 _ptr(scratch), s, v, _stream()), "sample")
    return out


def scatter_words(resident: torch.Tensor, pairs: torch.Tensor, count: int) -> None:
    """resident[pairs[2i]] = pairs[2i+1] for i < count (int32 arrays on the device; every index at most once)."""
    _i32(resident, "resident array"), _i32(pairs, "index/value pairs")
    if count < 0 or pairs.numel() < 2 * count:
        raise KernelError(f"{count} pairs do not fit in {pairs.numel()} words")
    check(lib().psb_scatter_words(resident.data_ptr(), pairs.data_ptr(), count, resident.numel(), _stream()), "scatter_words")


def step_prepare(records: torch.Tensor | None, kv_len: torch.Tensor | None, slots: torch.Tensor, rows: torch.Tensor | None,
                 out: torch.Tensor | None) -> None:
    """out[i, :] = rows[slots[i], :width] (the page table of a step from the rows that stay on the device, padded
    with -1 beyond their width), and records[slots[i]].position = kv_len[i].  Either half may be left out."""
    _i32(slots, "slots")
    b = slots.numel()
    num_slots = record_words = row_width = width = 0
    if records is not None:
        _i32(records, "slot records"), _i32(kv_len, "kv_len")
        if records.dim() != 2 or kv_len.numel() != b:
            raise KernelError("slot records must be [slots, words] and kv_len needs one entry per item")
        num_slots, record_words = records.shape
    if rows is not None:
        _i32(rows, "resident page table"), _i32(out, "page table of the step")
        if rows.dim() != 2 or out.dim() != 2 or out.shape[0] != b:
            raise KernelError(f"page tables must be [slots, pages] and [{b}, width], are {tuple(rows.shape)} and {tuple(out.shape)}")
        num_slots, row_width = rows.shape
        width = out.shape[1]
    if records is None and rows is None:
        return
    check(lib().psb_step_prepare(_ptr(records), record_words, _ptr(kv_len), slots.data_ptr(), _ptr(rows), row_width, _ptr(out),
                                 width, b, num_slots, _stream()), "step_prepare")
