"""bfloat16 fast paths: matrix products and attention on the tensor cores."""

from __future__ import annotations

from typing import Sequence

import torch

from .library import check, launch_counts, lib, stream_handle


# Tuning, set from measurements on B200 at Llama-1B sizes:
STREAM_M = 8        # rows up to which a layer's products run on the persistent streaming kernels (their limit is 16, but
                    # from 9 rows on they stream a second tile of rows beside every weight tile and the few-row tcgen05
                    # product, with the norm as a kernel of its own, is ahead: decode steps at Llama-1B sizes, context
                    # 4,096, ms a step with the streaming kernels / the few-row product: 8 requests 0.908 / 1.011,
                    # 9: 1.079 / 1.058, 10: 1.130 / 1.089, 12: 1.230 / 1.136, 14: 1.242 / 1.182, 16: 1.267 / 1.187)
STREAM_M_HEAD = 16  # ... and products with float32 output (the LM head, which the few-row product does not do)
USE_TCGEN05 = True  # products with more rows than STREAM_M: this library's tcgen05/TMEM/TMA kernel (else cuBLAS)
TCGEN05_MIN_TILES = 120  # ... when the kernel would cut the product into at least this many output tiles (128 rows by
                         # 256, 192 or 128 columns, whichever gets it done in the fewest, shortest rounds); smaller ones
                         # (a few dozen rows against a narrow matrix) leave most SMs idle without split-K and go to cuBLAS
TCGEN05_MIN_ROWS = 128   # ... and it has at least one full tile of rows: with 64 rows half of every instruction is padding
                         # (gate/up of 64 decoded tokens: 18 us against the library's 12.7 plus 2.4 for the activation)
USE_FEWROWS = True   # products with more rows than STREAM_M and at most FEWROWS_MAX[kind]: the kernel that puts the rows in
                     # the instruction's N dimension and shares the contraction out over a cluster (else cuBLAS).  Decode
                     # steps at Llama-1B sizes, context 4,096, ms a step, the library products with their norm, rotary
                     # and activation kernels / this kernel with a norm kernel between the products / this kernel with
                     # the norm carried by the products around it (FEWROWS_FUSE_NORM): 32 requests 1.681 / 1.610 / 1.533,
                     # 48: 2.372 / 2.361 / 1.922 (the last two after the key ranges of attention changed as well),
                     # 64: 2.335 / 2.420 / 2.342.  Alone, the kernel matches cuBLAS on the narrow matrices (O 5.9 us
                     # both at 64 rows, down 11.8 against 13.4) and loses on gate/up from 33 rows on (17.5 against
                     # 12.6 + 2.4 for the activation kernel: 128 one-tile CTAs that fill, stream and drain in step
                     # leave the memory idle at both ends); what it saves is the kernels between the products
FEWROWS_MAX = {"plain": 64, "gated": 64, "rope": 64}
WIDE_BELOW_TILES = 600   # matrices with fewer 16-row tiles than this get 16 warps per CTA instead of 8
TCGEN05_PREFILL_MIN_TOKENS = 64   # steps whose longest prompt portion has at least this many tokens run prefill attention
                                  # on the tcgen05 kernel (tiles of 128 rows); shorter portions fill too little of a tile
USE_TMA_DECODE = True     # decode attention: the kernel whose keys and values the TMA unit brings in (pages of 16 tokens
                          # or more), for key ranges of at least TMA_DECODE_MIN_RANGE keys; otherwise the one in which
                          # every lane copies its own pieces.  Measured at Llama-1B sizes, context 4,096, ms a decode step
                          # with the limit at 1,024 / 512 keys: 8 requests (ranges of 512 keys) 0.874 / 0.857 (means of
                          # three interleaved runs each, single runs from 0.833 to 0.878), 9 requests 1.086 / 1.049,
                          # 12: 1.168 / 1.103, 14: 1.220 / 1.149, 16 (ranges of 1,024 either way) 1.209 / 1.193; with 64
                          # requests (one range of 4,096 keys) 2.45 with this kernel and 2.67 with the other.  Below 512
                          # keys it loses: one request (ranges of 256 keys) 0.654 with the limit at 512, 0.676 at 256
TMA_DECODE_MIN_RANGE = 512
PREFILL_MIN_KEY_RANGES = 3        # ... at least this many: two ranges lose to one tile a CTA (512-token portions, 32 heads
                                  # of 64: 7.24 against 7.04 ms per 2,048 tokens)
PREFILL_MAX_KEY_RANGES = 8        # prefill attention with few CTAs: at most this many key ranges ...
PREFILL_MIN_BLOCKS_PER_RANGE = 4  # ... of at least this many key blocks each (a range pays for a partial result per row)
MIN_KEY_RANGE = 128       # split-KV: no key range shorter than this
DECODE_RANGE_OVERHEAD = 100  # split-KV: what a key range costs beside its keys, in keys
DECODE_MERGE_COST = 8        # split-KV: what one more range costs the merge, in keys (one request, us a step by range:
                             # 4,096 keys 643 at 128, 645 at 256, 669 at 512; 16,384 keys 767 at 128, 733 at 256, 780
                             # at 512, 949 at 1,024; 32,768 keys 950 at 128, 866 at 256, 833 at 512, 956 at 1,024)
DECODE_LANES_FACTOR = 1.2    # split-KV: the kernel for short ranges against the TMA-fed one, per key of a long range
DECODE_FORCE_CHUNK = 0   # tests and sweeps: the key range of split-KV decode attention, whatever the plan would choose
DECODE_CTAS_PER_SM = 4   # split-KV: CTAs of the decode kernels an SM holds at a time, heads of 64 (93 to 118 registers, 48 KB)
DECODE_CTAS_PER_SM_128 = 2  # ... and heads of 128 (168 registers, 64 to 96 KB).  Llama-3B sizes, 8 requests at 4,096 keys: ranges
                            # of 512 keys (two rounds) 2.349 ms a step, of 1,024 (one round) 2.311; 8B sizes 3.913 / 3.883
_OUT_CODE = {torch.float32: 0, torch.bfloat16: 1}


def small_m_ok(m: int, k: int, limit: int) -> bool:
    return 0 < m <= limit and k >= 32 and k % 32 == 0


def gemm_stream(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """The persistent streaming kernel itself (at most 16 rows, K a multiple of 32)."""
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty((m, n), dtype=out_dtype, device=x.device)
    check(lib().psb_gemm_stream(x.data_ptr(), w.data_ptr(), y.data_ptr(), _OUT_CODE[out_dtype], m, n, k, _sms(x.device),
                                stream_handle()), "gemm_stream")
    return y


def gemm_stream_gated(x: torch.Tensor, w_gate_up: torch.Tensor, activation: int = 0) -> torch.Tensor:
    m, k = x.shape
    inter = w_gate_up.shape[0] // 2
    act = torch.empty((m, inter), dtype=torch.bfloat16, device=x.device)
    check(lib().psb_gemm_stream_gated(x.data_ptr(), w_gate_up.data_ptr(), act.data_ptr(), m, inter, k, _sms(x.device),
                                      activation, stream_handle()), "gemm_stream_gated")
    return act


FUSE_NORM = True    # few rows: fold the residual sum and the RMSNorm in front of a product into the streaming kernel


def _norm_fusable(x, w: torch.Tensor, limit: int | None = None) -> bool:
    m, k = x.shape
    if m > min(16, STREAM_M if limit is None else limit):
        return False
    pending = x.pending
    if pending is not None and not isinstance(pending, torch.Tensor):
        return False  # a product that has not run yet: the few-row kernels take it
    return (FUSE_NORM and w.is_contiguous() and w.shape[1] == k and x.h.is_contiguous() and x.h.dtype == torch.float32
            and (pending is None or (pending.dtype == torch.bfloat16 and pending.is_contiguous() and pending.shape == x.h.shape))
            and k % 32 == 0 and 0 < m <= 16 and bool(lib().psb_gemm_stream_norm_supported(m, k)))


def norm_linear_bf16(x, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor | None:
    """rmsnorm(h + pending) @ w^T in the streaming kernel; None when that kernel does not take the shape.

    ``x`` is an ``ops.NormedRows`` that nobody has turned into a tensor yet.  The float32 stream after the sum goes to
    a new tensor (other CTAs still read the old one while the first CTA writes), which ``x`` is told of.
    """
    if out_dtype not in _OUT_CODE or not _norm_fusable(x, w, STREAM_M_HEAD if out_dtype == torch.float32 else STREAM_M):
        return None
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty((m, n), dtype=out_dtype, device=w.device)
    new_h = torch.empty_like(x.h) if (x.pending is not None and x.rows is None) else None
    check(lib().psb_gemm_stream_norm(x.h.data_ptr(), None if x.pending is None else x.pending.data_ptr(), x.gain.data_ptr(),
                                     None if x.rows is None else x.rows.data_ptr(), None if new_h is None else new_h.data_ptr(),
                                     w.data_ptr(), y.data_ptr(), _OUT_CODE[out_dtype], m, n, k, x.eps, _sms(w.device),
                                     stream_handle()), "gemm_stream_norm")
    x.fused(new_h)
    return y


def norm_qkv_rope_bf16(x, w_qkv, positions, token_item, cos, sin, table, kv, hq, hkv, d, page_size) -> torch.Tensor | None:
    """The streaming kernel with the residual sum and norm in front and rotation and append behind; None when it does
    not take the shape."""
    if not _norm_fusable(x, w_qkv):
        return None
    m, k = x.shape
    q = torch.empty((m, hq, d), dtype=torch.bfloat16, device=w_qkv.device)
    new_h = torch.empty_like(x.h) if x.pending is not None else None
    check(lib().psb_gemm_stream_norm_rope(
        x.h.data_ptr(), None if x.pending is None else x.pending.data_ptr(), x.gain.data_ptr(),
        None if new_h is None else new_h.data_ptr(), w_qkv.data_ptr(), m, k, x.eps, _sms(w_qkv.device), positions.data_ptr(),
        token_item.data_ptr(), table.data_ptr(), table.shape[1], None if cos is None else cos.data_ptr(),
        None if sin is None else sin.data_ptr(), kv.data_ptr(), q.data_ptr(), hq, hkv, d, page_size, kv.shape[0],
        0 if cos is None else cos.shape[0], stream_handle()), "gemm_stream_norm_rope")
    x.fused(new_h)
    return q


def norm_gated_linear_bf16(x, w_gate_up: torch.Tensor, activation: int = 0) -> torch.Tensor | None:
    """act(x Wg^T) * (x Wu^T) with x = rmsnorm(h + pending), all in the streaming kernel; None when it does not fit."""
    if w_gate_up.shape[0] % 2 or x.rows is not None or not _norm_fusable(x, w_gate_up):
        return None
    m, k = x.shape
    inter = w_gate_up.shape[0] // 2
    act = torch.empty((m, inter), dtype=torch.bfloat16, device=w_gate_up.device)
    new_h = torch.empty_like(x.h) if x.pending is not None else None
    check(lib().psb_gemm_stream_norm_gated(x.h.data_ptr(), None if x.pending is None else x.pending.data_ptr(), x.gain.data_ptr(),
                                           None if new_h is None else new_h.data_ptr(), w_gate_up.data_ptr(), act.data_ptr(),
                                           m, inter, k, x.eps, _sms(w_gate_up.device), activation,
                                           stream_handle()), "gemm_stream_norm_gated")
    x.fused(new_h)
    return act


def _fewrows_ok(x: torch.Tensor, w: torch.Tensor, kind: str = "plain") -> bool:
    m, k = x.shape
    return (USE_FEWROWS and STREAM_M < m <= FEWROWS_MAX[kind] and k >= 64 and k % 8 == 0 and x.is_contiguous() and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_fewrows(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x[M,K] @ w[N,K]^T -> bfloat16 for up to 64 rows: W as the tensor-core instruction's M operand, the contraction
    shared out over a thread-block cluster that adds its partial sums up through distributed shared memory."""
    m, k = x.shape
    y = torch.empty((m, w.shape[0]), dtype=torch.bfloat16, device=x.device)
    check(lib().psb_gemm_fewrows(x.data_ptr(), w.data_ptr(), y.data_ptr(), m, w.shape[0], k, stream_handle()), "gemm_fewrows")
    return y


def gemm_fewrows_gated(x: torch.Tensor, w_gate_up: torch.Tensor, activation: int = 0) -> torch.Tensor:
    m, k = x.shape
    inter = w_gate_up.shape[0] // 2
    act = torch.empty((m, inter), dtype=torch.bfloat16, device=x.device)
    check(lib().psb_gemm_fewrows_gated(x.data_ptr(), w_gate_up.data_ptr(), act.data_ptr(), m, inter, k, activation,
                                       stream_handle()), "gemm_fewrows_gated")
    return act


FEWROWS_FUSE_NORM = True  # few-row products around a norm: the one in front carries the residual sum, the gain and its share of
                          # the sums of squares in its epilogue, the one behind scales its sums (no norm kernel between them)
SSQ_PITCH = 64            # floats a tile in the array of shares (as in gemm_tcgen05_fewrows.cu)


def fewrows_lazy_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether a sublayer's last product may be handed on unrun: bfloat16, and so few rows that both the few-row
    products in front of and behind the next norm take them."""
    m = x.shape[0]
    return (FEWROWS_FUSE_NORM and USE_FEWROWS and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and STREAM_M < m <= min(FEWROWS_MAX.values()) and _fewrows_ok(x, w, "plain"))


def fewrows_add_norm(x: torch.Tensor, w: torch.Tensor, h: torch.Tensor, gain: torch.Tensor):
    """h += bfloat16(x @ w^T) in place (float32); returns (bfloat16(h * gain) [M, N], the tiles' shares of every row's
    sum(h^2) as float32 [tiles, 64]), or None when the few-row kernel does not take the shapes."""
    m, k = x.shape
    n = w.shape[0]
    if not (_fewrows_ok(x, w, "plain") and h.dtype == torch.float32 and h.is_contiguous() and h.shape == (m, n)
            and gain.dtype == torch.float32 and gain.numel() == n and h.data_ptr() % 16 == 0):
        return None
    gained = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    shares = torch.empty((-(-n // 128), SSQ_PITCH), dtype=torch.float32, device=x.device)
    check(lib().psb_gemm_fewrows_add_norm(x.data_ptr(), w.data_ptr(), h.data_ptr(), gain.data_ptr(), gained.data_ptr(),
                                          shares.data_ptr(), m, n, k, stream_handle()), "gemm_fewrows_add_norm")
    return gained, shares


def fewrows_behind_norm(x, w: torch.Tensor, kind: str, activation: int = 0, rope=None) -> torch.Tensor | None:
    """The product behind a norm whose input is still ``x`` (a NormedRows with a product pending in front of it), on the
    few-row kernel with the norm's factor applied to its sums; None when that does not apply (the caller goes on as usual).
    kind: "plain", "gated" or "rope" (then ``rope`` = positions, token_item, cos, sin, table, kv, hq, hkv, d, page_size)."""
    from .deferred import PendingProduct
    if not (FEWROWS_FUSE_NORM and isinstance(x.pending, PendingProduct) and x.rows is None and x.dtype == torch.bfloat16):
        return None
    m, k = x.shape
    if not (USE_FEWROWS and STREAM_M < m <= FEWROWS_MAX[kind] and k >= 64 and k % 8 == 0 and w.is_contiguous() and w.data_ptr() % 16 == 0):
        return None
    if kind == "rope":
        positions, token_item, cos, sin, table, kv, hq, hkv, d, page_size = rope
        if not (kv.is_contiguous() and (cos is None or (cos.is_contiguous() and sin.is_contiguous()))):
            return None
    raw = x.raw()
    if raw is None:
        return None
    gained, shares = raw
    parts = shares.shape[0]
    if kind == "plain":
        y = torch.empty((m, w.shape[0]), dtype=torch.bfloat16, device=w.device)
        check(lib().psb_gemm_fewrows_scaled(gained.data_ptr(), w.data_ptr(), y.data_ptr(), m, w.shape[0], k, shares.data_ptr(), parts,
                                            x.eps, stream_handle()), "gemm_fewrows")
        return y
    if kind == "gated":
        inter = w.shape[0] // 2
        act = torch.empty((m, inter), dtype=torch.bfloat16, device=w.device)
        check(lib().psb_gemm_fewrows_gated_scaled(gained.data_ptr(), w.data_ptr(), act.data_ptr(), m, inter, k, activation,
                                                  shares.data_ptr(), parts, x.eps, stream_handle()), "gemm_fewrows_gated")
        return act
    q = torch.empty((m, hq, d), dtype=torch.bfloat16, device=w.device)
    check(lib().psb_gemm_fewrows_rope_scaled(
        gained.data_ptr(), w.data_ptr(), m, k, positions.data_ptr(), token_item.data_ptr(), table.data_ptr(), table.shape[1],
        None if cos is None else cos.data_ptr(), None if sin is None else sin.data_ptr(), kv.data_ptr(), q.data_ptr(),
        hq, hkv, d, page_size, kv.shape[0], 0 if cos is None else cos.shape[0], shares.data_ptr(), parts, x.eps,
        stream_handle()), "gemm_fewrows_rope")
    return q


def _tcgen05_ok(x: torch.Tensor, w: torch.Tensor, kind: int = 0, head_dim: int = 0) -> bool:
    """kind: 0 plain, 1 gated (w holds gate and up rows), 2 the projection that rotates (heads of ``head_dim``)."""
    if not USE_TCGEN05:
        return False
    n_out = w.shape[0] // 2 if kind == 1 else w.shape[0]
    if x.shape[0] < TCGEN05_MIN_ROWS:
        return False
    tiles = lib().psb_gemm_tcgen05_tiles(x.shape[0], n_out, kind, head_dim, _sms(x.device))
    return (tiles >= TCGEN05_MIN_TILES and x.shape[1] % 8 == 0 and x.shape[1] >= 8 and x.is_contiguous() and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x[M,K] @ w[N,K]^T -> bfloat16, on tcgen05 tensor cores with TMEM accumulators, operands fed by TMA."""
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    check(lib().psb_gemm_tcgen05(x.data_ptr(), w.data_ptr(), y.data_ptr(), m, n, k, _sms(x.device),
                                 stream_handle()), "gemm_tcgen05")
    return y


def gemm_tcgen05_gated(x: torch.Tensor, w_gate_up: torch.Tensor, activation: int = 0) -> torch.Tensor:
    """act(x Wg^T) * (x Wu^T) -> bfloat16 [M, I], the activation applied in the product's epilogue."""
    m, k = x.shape
    inter = w_gate_up.shape[0] // 2
    act = torch.empty((m, inter), dtype=torch.bfloat16, device=x.device)
    check(lib().psb_gemm_tcgen05_gated(x.data_ptr(), w_gate_up.data_ptr(), act.data_ptr(), m, inter, k, _sms(x.device),
                                       activation, stream_handle()), "gemm_tcgen05_gated")
    return act


def tcgen05_qkv_rope_bf16(x: torch.Tensor, w_qkv, positions, token_item, cos, sin, table, kv, hq, hkv, d, page_size) -> torch.Tensor | None:
    """The projection of an attention layer for many tokens on the tcgen05 kernel, rotation and append to the pages in
    its epilogue (for a few dozen tokens: on the few-row kernel, which does the same); None when neither takes the shape."""
    if not (kv.is_contiguous() and (cos is None or (cos.is_contiguous() and sin.is_contiguous()))):
        return None
    m, k = x.shape
    if _fewrows_ok(x, w_qkv, "rope"):
        q = torch.empty((m, hq, d), dtype=torch.bfloat16, device=x.device)
        check(lib().psb_gemm_fewrows_rope(
            x.data_ptr(), w_qkv.data_ptr(), m, k, positions.data_ptr(), token_item.data_ptr(), table.data_ptr(), table.shape[1],
            None if cos is None else cos.data_ptr(), None if sin is None else sin.data_ptr(), kv.data_ptr(), q.data_ptr(),
            hq, hkv, d, page_size, kv.shape[0], 0 if cos is None else cos.shape[0], stream_handle()), "gemm_fewrows_rope")
        return q
    if not _tcgen05_ok(x, w_qkv, 2, d):
        return None
    q = torch.empty((m, hq, d), dtype=torch.bfloat16, device=x.device)
    check(lib().psb_gemm_tcgen05_rope(
        x.data_ptr(), w_qkv.data_ptr(), m, k, _sms(x.device), positions.data_ptr(), token_item.data_ptr(), table.data_ptr(),
        table.shape[1], None if cos is None else cos.data_ptr(), None if sin is None else sin.data_ptr(), kv.data_ptr(),
        q.data_ptr(), hq, hkv, d, page_size, kv.shape[0], 0 if cos is None else cos.shape[0], stream_handle()),
        "gemm_tcgen05_rope")
    return q


def linear_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x[M,K] @ w[N,K]^T for bfloat16 operands, float32 accumulation.

    Up to STREAM_M rows (decode): the weight-streaming kernel of this library.  A few dozen rows: its few-row tcgen05
    kernel.  Prefill-sized products with bfloat16 output: its tcgen05 kernel.  What lies between (and outputs in
    float32 with many rows) goes to the library
    product (cuBLAS through torch), which is where the reference calls F.linear for everything
    (prefixserve/model/llama.py:113-126).
    """
    m, k = x.shape
    if out_dtype in _OUT_CODE and x.is_contiguous() and w.is_contiguous():
        if small_m_ok(m, k, min(STREAM_M_HEAD if out_dtype == torch.float32 else STREAM_M, 16)):
            return gemm_stream(x, w, out_dtype)
        if out_dtype == torch.bfloat16 and _fewrows_ok(x, w):
            return gemm_fewrows(x, w)
        if out_dtype == torch.bfloat16 and m > 0 and _tcgen05_ok(x, w):
            return gemm_tcgen05(x, w)
    if out_dtype == torch.float32:  # logits of many rows: the sums leave the library in float32, never rounded to bfloat16
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    y = torch.nn.functional.linear(x, w)
    return y if out_dtype == y.dtype else y.to(out_dtype)


def gated_linear_bf16(x: torch.Tensor, w_gate_up: torch.Tensor, activation: int = 0) -> torch.Tensor | None:
    """act(x Wg^T) * (x Wu^T) in one kernel (few rows: the streaming product; many: the tcgen05 product); None when
    neither takes the shape."""
    m, k = x.shape
    if w_gate_up.shape[0] % 2 or not (x.is_contiguous() and w_gate_up.is_contiguous()):
        return None
    if small_m_ok(m, k, min(STREAM_M, 16)):
        return gemm_stream_gated(x, w_gate_up, activation)
    if _fewrows_ok(x, w_gate_up, "gated"):
        return gemm_fewrows_gated(x, w_gate_up, activation)
    if m > STREAM_M and _tcgen05_ok(x, w_gate_up, 1):
        return gemm_tcgen05_gated(x, w_gate_up, activation)
    return None


_sm_count: dict[int, int] = {}
_scratch: dict[tuple[int, str], list[torch.Tensor]] = {}


def _sms(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _sm_count:
        _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count[idx]


def _scratch_buffer(device: torch.device, name: str, numel: int) -> torch.Tensor:
    """A float32 buffer that lives as long as the process (split-KV partial results).  When a larger one is needed a
    new one is made and the old ones are KEPT: captured steps have their address baked in and go on using them."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), name)
    held = _scratch.setdefault(key, [])
    if not held or held[-1].numel() < numel:
        held.append(torch.empty(max(numel, 1 << 16), dtype=torch.float32, device=device))
    return held[-1]


def attention_bf16_supported(head_dim: int, page_size: int) -> bool:
    return head_dim in (64, 128) and page_size >= 16 and page_size & (page_size - 1) == 0


def _decode_key_range(pairs: int, longest: int, sms: int, tma_kernel: bool, ctas_per_sm: int | None = None) -> int:
    """The key range of split-KV decode attention for ``pairs`` (request, key/value head) pairs of up to ``longest``
    keys.  An SM runs ``ctas_per_sm`` CTAs at a time (DECODE_CTAS_PER_SM for heads of 64), each at its own pace (a CTA alone on an SM is no faster), so a
    launch takes as many rounds as its CTAs fill those slots, each as long as a range plus a fixed share: one round of
    the shortest ranges that fit into it, unless that leaves many slots empty and several rounds of shorter ranges
    come out ahead (48 requests with 8 heads at 4,096 keys: one round of 384 whole sequences against two rounds of
    1,152 thirds, measured 2.34 against 2.00 ms a step).  Ranges below TMA_DECODE_MIN_RANGE go to the kernel whose
    lanes copy for themselves, which is slower on long ranges (111 against 93 us at 64 requests)."""
    slots = (ctas_per_sm or DECODE_CTAS_PER_SM) * sms
    pairs = max(1, pairs)
    most = max(1, min(-(-longest // MIN_KEY_RANGE), 4 * (slots // pairs + 1)))  # shorter ranges cost more to merge than they save
    fewest = None   # (rounds, cost, range) of the best plan among those with the fewest rounds
    best = None     # ... and of the best plan of all
    for splits in range(1, most + 1):
        chunk = -(-(-(-longest // splits)) // 64) * 64
        rounds = -(-(pairs * -(-longest // chunk)) // slots)
        cost = rounds * (chunk + DECODE_RANGE_OVERHEAD) * (1.0 if tma_kernel and chunk >= TMA_DECODE_MIN_RANGE else DECODE_LANES_FACTOR)
        cost += DECODE_MERGE_COST * -(-longest // chunk)  # the kernel that joins the ranges reads one partial result a range
        plan = (rounds, cost, chunk)
        if fewest is None or rounds < fewest[0] or (rounds == fewest[0] and cost < fewest[1]):
            fewest = plan
        if best is None or cost < best[1]:
            best = plan
    # more rounds only for a clear gain, 3 % for every round more: the estimate is rough (Llama-3B sizes, 8 requests at
    # 16,384 keys: two rounds of 1,856 keys are estimated 7 % ahead of one round of 4,096 and measure 4.21 against 4.41 ms)
    if best[0] > fewest[0] and best[1] > (1.0 - 0.03 * (best[0] - fewest[0])) * fewest[1]:
        best = fewest
    return best[2]


def _attention_plan(new_tokens: Sequence[int], kv_lens: Sequence[int], window: int, group: int, hkv: int, d: int, page: int,
                    sms: int, static_kv_len: int | None) -> dict:
    """Launch shapes of a step's attention, from the host copies of the items' lengths.  The same for every layer with
    the same head counts and window, so a step works it out once."""
    hq_total = group * hkv
    b = len(new_tokens)
    singles = [kvl for n, kvl in zip(new_tokens, kv_lens) if n == 1]
    if static_kv_len is not None:  # a captured step: its single tokens may later sit at any length up to this one
        singles = [static_kv_len] * len(singles)
    plan = {"b": b, "use_decode": bool(singles) and group <= 16}
    if plan["use_decode"]:
        if window and static_kv_len is not None:
            # a captured step serves every length up to static_kv_len: the span from the 16-aligned start of the
            # window to the newest key depends on (length - window) mod 16 and reaches window + 15
            longest = min(static_kv_len, window + 15)
        elif window:  # keys a decode item reads, from the 16-aligned start of its window
            longest = max(kvl - (max(0, kvl - window) // 16) * 16 for kvl in singles)
        else:
            longest = max(singles)
        plan["chunk"] = DECODE_FORCE_CHUNK or _decode_key_range(b * hkv, longest, sms, bool(
            USE_TMA_DECODE and lib().psb_attention_decode_tma_supported(hq_total, hkv, d, page)),
            DECODE_CTAS_PER_SM if d <= 64 else DECODE_CTAS_PER_SM_128)
        plan["max_splits"] = -(-longest // plan["chunk"])
        plan["all_single"] = 1 if len(singles) == b else 0
    portions = [n for n in new_tokens if not (plan["use_decode"] and n == 1)]
    plan["tcgen05"] = bool(USE_TCGEN05 and portions and max(portions) >= TCGEN05_PREFILL_MIN_TOKENS
                           and lib().psb_attention_prefill_tcgen05_supported(d, page))
    if plan["tcgen05"]:
        # a CTA takes 256 rows of one head as two tiles that fill each other's waits; when that leaves more than half
        # of the SMs without a CTA (a few hundred new tokens), one tile each and twice the CTAs (measured at 32 heads:
        # 512-token portions 7.29 -> 7.04 ms per 2,048 tokens, 1,024-token portions would lose)
        per_cta = lib().psb_attention_prefill_tcgen05_rows_per_cta()
        ctas = hq_total * sum(-(-n // per_cta) for n in portions)
        plan["kv_splits"] = 1
        if ctas <= sms // 2:
            # few CTAs: cut the keys into ranges if the portions' contexts are long enough (at least
            # PREFILL_MIN_BLOCKS_PER_RANGE blocks a range), else give every CTA one tile instead of two
            longest = static_kv_len if static_kv_len is not None else max(kvl for n, kvl in zip(new_tokens, kv_lens) if not (plan["use_decode"] and n == 1))
            blocks = -(-longest // (128 if d == 64 else 64))
            splits = min(PREFILL_MAX_KEY_RANGES, sms // ctas, blocks // PREFILL_MIN_BLOCKS_PER_RANGE)
            if splits >= PREFILL_MIN_KEY_RANGES:
                plan["kv_splits"] = splits
            else:
                per_cta //= 2
        plan["rows_per_cta"] = per_cta
        plan["pairs"] = sum(-(-n // per_cta) for n in portions)
    else:
        rows = lib().psb_attention_prefill_rows_per_cta(d)
        plan["tiles"] = sum(-(-(n * group) // rows) for n in portions)
    return plan


def attention_bf16(q: torch.Tensor, kv: torch.Tensor, table: torch.Tensor, item_start: torch.Tensor, kv_len: torch.Tensor,
                   new_tokens: Sequence[int] | None, kv_lens: Sequence[int] | None, *, window: int | None, scale: float,
                   static_kv_len: int | None = None, plans: dict | None = None, items=None,
                   token_item: torch.Tensor | None = None) -> torch.Tensor | None:
    """Tensor-core attention for a step.  ``new_tokens``/``kv_lens`` are the host copies of what ``item_start`` and
    ``kv_len`` hold on the device (or ``items`` with ``.start``/``.end``, read only when no plan is cached yet).
    Returns None when no kernel here takes the shape (the caller falls back).  ``plans``: a dict that lives as long as
    the step; layers with the same shape reuse the launch plan the first of them worked out.

    With ``static_kv_len`` (a step that is being captured for replay) the launch shapes are derived from that
    length instead of the items' own, so they are the same for every later step of the same batch size."""
    t, hq, d = q.shape
    _, _, hkv, page, _ = kv.shape
    if not attention_bf16_supported(d, page):
        return None
    group = hq // hkv
    w = int(window or 0)
    key = ("attention plan", w, hq, hkv, d, page)
    plan = plans.get(key) if plans is not None else None
    if plan is None:
        if new_tokens is None:
            new_tokens, kv_lens = [it.end - it.start for it in items], [it.end for it in items]
        plan = _attention_plan(new_tokens, kv_lens, w, group, hkv, d, page, _sms(q.device), static_kv_len)
        if plans is not None:
            plans[key] = plan
    out = torch.empty((t, hq * d), dtype=torch.bfloat16, device=q.device)
    stream = stream_handle()
    b = plan["b"]
    if plan["use_decode"]:
        chunk, max_splits = plan["chunk"], plan["max_splits"]
        part_o = part_ml = None
        if max_splits > 1:
            part_o = _scratch_buffer(q.device, "attn_o", b * hq * max_splits * d)
            part_ml = _scratch_buffer(q.device, "attn_ml", b * hq * max_splits * 2)
        po = part_o.data_ptr() if part_o is not None else None
        pm = part_ml.data_ptr() if part_ml is not None else None
        if (USE_TMA_DECODE and chunk >= TMA_DECODE_MIN_RANGE and kv.is_contiguous()
                and lib().psb_attention_decode_tma_supported(hq, hkv, d, page)):
            check(lib().psb_attention_decode_tma_bf16(
                q.data_ptr(), kv.data_ptr(), table.data_ptr(), table.shape[1], item_start.data_ptr(), kv_len.data_ptr(),
                out.data_ptr(), po, pm, b, hq, hkv, d, page, kv.shape[0], w, float(scale), chunk, max_splits,
                plan["all_single"], stream), "attention_decode")
            launch_counts["attention_decode_tma"] += 1  # the same step of the model, by which kernel
            if max_splits > 1:
                check(lib().psb_attention_decode_merge_bf16(po, pm, item_start.data_ptr(), kv_len.data_ptr(), out.data_ptr(), b, hq, d,
                                                            w, chunk, max_splits, plan["all_single"], stream), "attention_merge")
        else:
            check(lib().psb_attention_decode_bf16(
                q.data_ptr(), kv.data_ptr(), table.data_ptr(), table.shape[1], item_start.data_ptr(), kv_len.data_ptr(),
                out.data_ptr(), po, pm, b, hq, hkv, d, page, w, float(scale), chunk, max_splits,
                plan["all_single"], stream), "attention_decode")
    if plan["tcgen05"] and q.is_contiguous() and kv.is_contiguous():
        splits = plan["kv_splits"] if token_item is not None else 1
        po = pm = None
        if splits > 1:
            po = _scratch_buffer(q.device, "prefill_o", t * hq * splits * d).data_ptr()
            pm = _scratch_buffer(q.device, "prefill_ml", t * hq * splits * 2).data_ptr()
        check(lib().psb_attention_prefill_tcgen05(
            q.data_ptr(), kv.data_ptr(), table.data_ptr(), table.shape[1], item_start.data_ptr(), kv_len.data_ptr(),
            out.data_ptr(), b, plan["pairs"], t, hq, hkv, d, page, kv.shape[0], w, float(scale),
            1 if plan["use_decode"] else 0, plan["rows_per_cta"], splits, po, pm,
            token_item.data_ptr() if token_item is not None else None, stream), "attention_prefill_tcgen05")
        return out
    tiles = plan.get("tiles")
    if tiles is None:  # planned for the tcgen05 kernel, which these tensors' layout rules out
        rows = lib().psb_attention_prefill_rows_per_cta(d)
        new_tokens = new_tokens if new_tokens is not None else [it.end - it.start for it in items]
        tiles = sum(-(-(n * group) // rows) for n in new_tokens if not (plan["use_decode"] and n == 1))
    if tiles:
        check(lib().psb_attention_prefill_bf16(
            q.data_ptr(), kv.data_ptr(), table.data_ptr(), table.shape[1], item_start.data_ptr(), kv_len.data_ptr(),
            out.data_ptr(), b, tiles, hq, hkv, d, page, w, float(scale), 1 if plan["use_decode"] else 0, stream), "attention_prefill")
    return out
