"""Loads the CUDA kernel library and declares its C entry points.

There is no fallback: if the library cannot be built or loaded, or no CUDA
device is present, importing an op raises.
"""

from __future__ import annotations

import ctypes
import os
from collections import Counter
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from ..build import ensure_kernels


class KernelError(RuntimeError):
    """A kernel refused its arguments or the launch failed."""


_lib: ctypes.CDLL | None = None

P, I, L, F = c_void_p, c_int, c_int64, c_float

# name -> argument types (every entry point returns an int status, 0 = ok)
_SIGNATURES: dict[str, list] = {
    # (ids, table, table_dtype, out_f32, T, H, V, stream)
    "psb_embedding": [P, P, I, P, I, I, I, P],
    # (h, delta, delta_dtype, weight, rows, x, x_dtype, n_rows, H, eps, update_h, stream)
    "psb_add_rmsnorm": [P, P, I, P, P, P, I, I, I, F, I, P],
    # (a, a_dtype, w, w_dtype, c, c_dtype, M, N, K, lda, ldw, ldc, accumulate, stream)
    "psb_gemm_nt": [P, I, P, I, P, I, I, I, I, L, L, L, I, P],
    # (qkv, dtype, positions, token_item, cos, sin, table, table_width, kv, kv_dtype, q_out,
    #  T, hq, hkv, D, page_size, num_pages, max_positions, rotate, write_kv, paired, rotary_dim, interleaved, stream)
    "psb_rope_append": [P, I, P, P, P, P, P, I, P, I, P, I, I, I, I, I, I, I, I, I, I, I, I, P],
    # (h_in, pending, gain, h_out, W, M, K, eps, sms, positions, token_item, table, table_width, cos, sin, kv, q_out,
    #  hq, hkv, D, page_size, num_pages, max_positions, stream)
    "psb_gemm_stream_norm_rope": [P, P, P, P, P, I, I, F, I, P, P, P, I, P, P, P, P, I, I, I, I, I, I, P],
    # (q, dtype, kv, kv_dtype, table, table_width, positions, token_item, out, T, hq, hkv, D, page_size, window,
    #  scale, stream)
    "psb_attention_generic": [P, I, P, I, P, I, P, P, P, I, I, I, I, I, I, F, P],
    # (gate_up, dtype, out, T, I, activation, stream)
    "psb_silu_mul": [P, I, P, I, I, I, P],
    # (h, delta, delta_dtype, total, stream)
    "psb_residual_add": [P, P, I, L, P],
    # (q, kv, table, table_width, item_start, kv_len, out, num_items, num_tiles, hq, hkv, D, page_size, window, scale,
    #  skip_single, stream)
    "psb_attention_prefill_bf16": [P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, P],
    # (D) -> rows per CTA
    "psb_attention_prefill_rows_per_cta": [I],
    # (D, page_size) -> 1 if the tcgen05 prefill attention takes them
    "psb_attention_prefill_tcgen05_supported": [I, I],
    # () -> rows per CTA
    "psb_attention_prefill_tcgen05_rows_per_cta": [],
    # (q, kv, table, table_width, item_start, kv_len, out, num_items, num_pairs, T, hq, hkv, D, page_size, num_pages,
    #  window, scale, skip_single, rows_per_cta, kv_splits, part_o, part_ml, token_item, stream)
    "psb_attention_prefill_tcgen05": [P, P, P, I, P, P, P, I, I, I, I, I, I, I, L, I, F, I, I, I, P, P, P, P],
    # () -> 0 while no bounded wait of the tcgen05 attention kernel has ever run out
    "psb_attention_tcgen05_status": [],
    # (q, kv, table, table_width, item_start, kv_len, out, part_o, part_ml, num_items, hq, hkv, D, page_size, window,
    #  scale, chunk, max_splits, all_single, stream)
    "psb_attention_decode_bf16": [P, P, P, I, P, P, P, P, P, I, I, I, I, I, I, F, I, I, I, P],
    # (hq, hkv, D, page_size) -> 1 if the TMA-fed decode attention takes the shape
    "psb_attention_decode_tma_supported": [I, I, I, I],
    # (q, kv, table, table_width, item_start, kv_len, out, part_o, part_ml, num_items, hq, hkv, D, page_size, num_pages,
    #  window, scale, chunk, max_splits, all_single, stream)
    "psb_attention_decode_tma_bf16": [P, P, P, I, P, P, P, P, P, I, I, I, I, I, L, I, F, I, I, I, P],
    "psb_attention_decode_tma_status": [],
    # (part_o, part_ml, item_start, kv_len, out, num_items, hq, D, window, chunk, max_splits, all_single, stream)
    "psb_attention_decode_merge_bf16": [P, P, P, P, P, I, I, I, I, I, I, I, P],
    # (x, W, y, out_dtype, M, N, K, sms, stream)
    "psb_gemm_stream": [P, P, P, I, I, I, I, I, P],
    # (x, W, act, M, I, K, sms, activation, stream)
    "psb_gemm_stream_gated": [P, P, P, I, I, I, I, I, P],
    # (M, K) -> 1 if the norm-fused streaming product takes the shape
    "psb_gemm_stream_norm_supported": [I, I],
    # (h_in, pending, gain, rows, h_out, W, y, out_dtype, M, N, K, eps, sms, stream)
    "psb_gemm_stream_norm": [P, P, P, P, P, P, P, I, I, I, I, F, I, P],
    # (h_in, pending, gain, h_out, W, act, M, I, K, eps, sms, activation, stream)
    "psb_gemm_stream_norm_gated": [P, P, P, P, P, P, I, I, I, F, I, I, P],
    # (a, w, c, M, N, K, sms, stream)
    "psb_gemm_tcgen05": [P, P, P, I, I, I, I, P],
    # (a, w, act, M, I, K, sms, activation, stream)
    "psb_gemm_tcgen05_gated": [P, P, P, I, I, I, I, I, P],
    "psb_gemm_tcgen05_tile_width": [I],
    # (M, N_out, kind, D, sms) -> output tiles at the width the kernel would choose
    "psb_gemm_tcgen05_tiles": [I, I, I, I, I],
    "psb_gemm_tcgen05_rope": [P, P, I, I, I, P, P, P, I, P, P, P, P, I, I, I, I, I, I, P],
    # () -> 0 while no bounded wait of the tcgen05 kernel has ever run out
    "psb_tcgen05_status": [],
    # the product for a few dozen rows (up to 64): (a, w, c, M, N, K, stream)
    "psb_gemm_fewrows": [P, P, P, I, I, I, P],
    # (a, w, act, M, I, K, activation, stream)
    "psb_gemm_fewrows_gated": [P, P, P, I, I, I, I, P],
    # (a, w, M, K, positions, token_item, table, table_width, cos, sin, kv, q_out, hq, hkv, D, page_size, num_pages, max_positions, stream)
    "psb_gemm_fewrows_rope": [P, P, I, I, P, P, P, I, P, P, P, P, I, I, I, I, I, I, P],
    # behind a norm: (..., ssq_in, ssq_parts, eps, stream)
    "psb_gemm_fewrows_scaled": [P, P, P, I, I, I, P, I, F, P],
    "psb_gemm_fewrows_gated_scaled": [P, P, P, I, I, I, I, P, I, F, P],
    "psb_gemm_fewrows_rope_scaled": [P, P, I, I, P, P, P, I, P, P, P, P, I, I, I, I, I, I, P, I, F, P],
    # in front of a norm: (a, w, stream float32 in/out, gain, gained bf16 out, ssq_out, M, N, K, stream)
    "psb_gemm_fewrows_add_norm": [P, P, P, P, P, P, I, I, I, P],
    "psb_gemm_fewrows_splits": [I],
    "psb_gemm_fewrows_status": [],
    # (logits, temperature, seed, position, out, scratch, S, V, stream)
    "psb_sample": [P, P, P, P, P, P, I, I, P],
    # (logits, records, row_slot, record_words, out, scratch, S, V, stream)
    "psb_sample_slots": [P, P, P, I, P, P, I, I, P],
    # (resident, pairs, n, limit, stream)
    "psb_scatter_words": [P, P, I, I, P],
    # (records, record_words, kv_len, slots, rows, row_width, out, width, num_items, num_slots, stream)
    "psb_step_prepare": [P, I, P, P, P, I, P, I, I, I, P],
    # (limit, who, out int32[3], stream)
    "psb_selftest_bounded_wait": [I, I, P, P],
    # (bytes, void** out) / (pointer)
    "psb_pool_alloc": [L, ctypes.POINTER(c_void_p)],
    "psb_pool_free": [P],
    # (S, V) -> bytes of scratch psb_sample wants
    "psb_sample_scratch_bytes": [I, I],
}


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = ensure_kernels()
        handle = ctypes.CDLL(str(path))
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        handle.psb_sample_scratch_bytes.restype = ctypes.c_longlong
        handle.psb_last_error.restype = ctypes.c_char_p
        handle.psb_last_error.argtypes = []
        handle.psb_set_pdl.argtypes = [c_int]
        handle.psb_set_pdl.restype = None
        handle.psb_get_pdl.argtypes = []
        handle.psb_get_pdl.restype = c_int
        if os.environ.get("PSB200_PDL", "1") == "0":  # plain stream order between kernels (for comparisons)
            handle.psb_set_pdl(0)
        _lib = handle
    return _lib


def set_pdl(on: bool) -> None:
    """Whether kernels are launched so that each may overlap its start with the end of its predecessor
    (programmatic dependent launch).  Graphs captured earlier keep the mode they were captured with."""
    lib().psb_set_pdl(1 if on else 0)


def pdl_enabled() -> bool:
    return bool(lib().psb_get_pdl())


_pinned_stream: int | None = None


def stream_handle() -> int:
    """The raw handle of the stream kernels are launched on: torch's current stream, looked up on every call unless a
    step has pinned it (``pinned_stream``): the lookup costs more host time than the launch it serves."""
    if _pinned_stream is not None:
        return _pinned_stream
    return torch.cuda.current_stream().cuda_stream


class pinned_stream:
    """Within the block, ``stream_handle()`` is torch's current stream as it was at entry.  For code that launches many
    kernels on one stream and does not switch streams itself (a step of the engine, the capture of one)."""

    def __enter__(self):
        global _pinned_stream
        self._before = _pinned_stream
        _pinned_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _pinned_stream
        _pinned_stream = self._before


def tcgen05_status() -> int:
    """0 unless a bounded wait inside a tcgen05 kernel ever gave up (then its results are void). Synchronises.

    The product's code sits in the low byte, prefill attention's in the next, the TMA-fed decode attention's in the
    third, the few-row product's in the fourth."""
    return (int(lib().psb_tcgen05_status()) | (int(lib().psb_attention_tcgen05_status()) << 8)
            | (int(lib().psb_attention_decode_tma_status()) << 16) | (int(lib().psb_gemm_fewrows_status()) << 24))


def declare(name: str, argtypes: list) -> None:
    """Adds an entry point (used by kernels that arrive in later files)."""
    _SIGNATURES[name] = argtypes
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int


launches = 0  # kernels of this library launched so far (benchmarks report the difference over a timed region)
launch_counts: Counter = Counter()  # the same by entry point ("attention_decode", "gemm_tcgen05", ...)


def check(status: int, what: str) -> None:
    global launches
    launches += 1
    launch_counts[what] += 1
    if status != 0:
        detail = lib().psb_last_error().decode(errors="replace")
        raise KernelError(f"{what}: {detail} (status {status})")


_parked: list[tuple[int, torch.device]] = []  # pool memory waiting to be freed (see DevicePool.free)


def _free_parked() -> None:
    if _lib is None or not _parked:
        return
    try:
        if torch.cuda.is_current_stream_capturing():
            return
    except Exception:  # noqa: BLE001  (interpreter shutdown)
        return
    while _parked:
        ptr, device = _parked.pop()
        with torch.cuda.device(device):
            _lib.psb_pool_free(c_void_p(ptr))


class DevicePool:
    """Device memory for cache pages, allocated and freed by the kernel library itself (not by torch's caching
    allocator): the address never moves and the bytes are given back the moment the owner goes.  ``tensor`` views
    the memory without copying; the views must not outlive the pool."""

    def __init__(self, nbytes: int, device: torch.device) -> None:
        self.nbytes, self.device = int(nbytes), torch.device(device)
        self.ptr = 0
        _free_parked()
        with torch.cuda.device(self.device):
            out = c_void_p()
            status = lib().psb_pool_alloc(self.nbytes, ctypes.byref(out))
            if status != 0:
                raise KernelError("pool: " + lib().psb_last_error().decode(errors="replace"))
            self.ptr = int(out.value)

    def tensor(self, shape: tuple, dtype: torch.dtype) -> torch.Tensor:
        typestr = {torch.bfloat16: "<u2", torch.float32: "<f4", torch.float16: "<f2"}[dtype]
        count = 1
        for n in shape:
            count *= int(n)
        if count * torch.empty((), dtype=dtype).element_size() > self.nbytes:
            raise KernelError(f"pool of {self.nbytes} bytes cannot hold a {dtype} tensor of shape {tuple(shape)}")

        class _Span:  # what torch needs to wrap foreign device memory; it keeps the pool alive while a view of it lives
            owner = self
            __cuda_array_interface__ = {"shape": tuple(int(n) for n in shape), "typestr": typestr, "data": (self.ptr, False),
                                        "version": 2, "strides": None}
        raw = torch.as_tensor(_Span(), device=self.device)
        return raw.view(dtype) if raw.dtype != dtype else raw

    def free(self) -> None:
        """Gives the memory back.  Freeing device memory waits for the device, which a stream capture in progress does
        not survive; a pool that dies during one (the collector may run its finaliser at any moment) is parked and
        freed by the next pool that is made or freed outside a capture."""
        if self.ptr:
            _parked.append((self.ptr, self.device))
            self.ptr = 0
        _free_parked()

    def __del__(self) -> None:
        try:
            self.free()
        except Exception:  # noqa: BLE001  (interpreter shutdown)
            pass
