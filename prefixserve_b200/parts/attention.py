"""Grouped-query attention over the paged cache.

q, k, v come from one fused projection; queries and keys are rotated by
absolute position and the new keys and values are appended to the request's
pages in the same kernel; attention then reads only from the pages; one output
projection follows (prefixserve/model/llama.py:113-117,
prefixserve/model/attention.py:68-121).  Sizes, the position encoding and an
optional window are parameters.  A call that only reads another call's cache
entry (``CacheView.writes`` false) has no key/value projection.
"""

from __future__ import annotations

import math

import torch

from .. import ops
from .base import CacheNeed, CacheView, Mixer, PagedKV, ParamSpec, StepContext
from .registry import make, register_mixer


class Attention(Mixer):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs
    takes_deferred_input = True  # x goes to one product only, which may do the norm in front of it itself

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden_size"])
        self.hq = int(params["num_heads"])
        self.hkv = int(params["num_kv_heads"])
        self.d = int(params["head_dim"])
        self.window = params.get("window")
        self.own_kv = bool(params.get("own_kv", True))
        self.scale = float(params.get("scale") or 1.0 / math.sqrt(self.d))
        if self.hq % self.hkv:
            raise ValueError(f"{self.hq} query heads cannot share {self.hkv} key/value heads")
        self.position = make("position", params["position"])
        # what the position part says about its rotation (a part that does not rotate says nothing)
        self.rotary_dim = int(getattr(self.position, "rotary_dim", None) or self.d)
        self.interleaved = getattr(self.position, "layout", "half") == "interleaved"
        # With head sizes that are multiples of 16, and a rotation (if any) of the split-half kind over the whole head,
        # queries and keys are kept in the pair-interleaved element order (see load()); any other rotation keeps the
        # natural order and goes through the general rotary kernel.
        self.paired = self.d % 16 == 0 and self.rotary_dim == self.d and not self.interleaved
        self.w_qkv: torch.Tensor | None = None
        self.w_o: torch.Tensor | None = None

    def param_specs(self):
        q, kv = self.hq * self.d, self.hkv * self.d
        specs = {"q_proj": ParamSpec((q, self.hidden))}
        if self.own_kv:
            specs["k_proj"] = ParamSpec((kv, self.hidden))
            specs["v_proj"] = ParamSpec((kv, self.hidden))
        specs["o_proj"] = ParamSpec((self.hidden, q))
        return specs

    def cache_need(self):
        return CacheNeed(paged=PagedKV(self.hkv, self.d, self.window, "paired" if self.paired else "natural"))

    def load(self, tensors, *, compute_dtype, device):
        pieces = [tensors["q_proj"]]
        if self.own_kv:
            pieces += [tensors["k_proj"], tensors["v_proj"]]
        # one matrix for the three projections (rows: queries, keys, values)
        dtype = torch.float32 if any(p.dtype == torch.float32 for p in pieces) else pieces[0].dtype
        pieces = [p.to(dtype) for p in pieces]
        # With head sizes that are multiples of 16 the rows of every query and key head are reordered so that each run
        # of 16 holds 8 elements of the head's first half and the 8 they are rotated with: the decode kernel that
        # computes a 16-row tile of this product can then rotate and store it itself.  Queries and keys keep that
        # element order all the way (scores do not depend on it); every attention part does this, rotating or not, so
        # that a layer which reads another layer's keys meets the order it uses itself (the order is part of the cache
        # need, so a reader that would disagree is refused when the model is put together).
        if self.paired:
            order = torch.tensor(ops.pair_interleaved_order(self.d), device=pieces[0].device)
            for at in range(2 if self.own_kv else 1):
                heads = pieces[at].shape[0] // self.d
                pieces[at] = pieces[at].view(heads, self.d, -1)[:, order, :].reshape(heads * self.d, -1)
        self.w_qkv = torch.cat(pieces, dim=0).contiguous()
        self.w_o = tensors["o_proj"].contiguous()

    def prepare(self, *, max_positions, compute_dtype, device):
        self.position.prepare(max_positions=max_positions, compute_dtype=compute_dtype, device=device)

    def forward(self, x, ctx: StepContext, cache: CacheView):
        if cache.writes != self.own_kv:
            raise RuntimeError("an attention part with its own keys and values must write its cache entry, and only such a part may")
        table = ctx.block_tables[cache.group]
        q = None
        if self.paired and self.own_kv and isinstance(x, ops.NormedRows):  # few tokens: projection, rotation, append in one
            q = ops.qkv_rope_append(x, self.w_qkv, ctx.positions, ctx.token_item, self.position.cos, self.position.sin, table,
                                    cache.kv, num_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.d,
                                    page_size=cache.page_size)
        if q is None:
            qkv = ops.linear(x, self.w_qkv)
            q = ops.rope_append(qkv, ctx.positions, ctx.token_item, self.position.cos, self.position.sin, table, cache.kv,
                                num_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.d, page_size=cache.page_size,
                                write_kv=self.own_kv, paired=self.paired, rotary_dim=self.rotary_dim,
                                interleaved=self.interleaved)
        o = ops.attention(q, cache.kv, table, ctx.positions, ctx.token_item, window=self.window, scale=self.scale, ctx=ctx)
        return ops.last_product(o, self.w_o, ctx)  # may be handed on unrun: the next norm's kernels take it from there


register_mixer("attention", Attention, replace=True)
