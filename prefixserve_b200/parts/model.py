"""A decoder assembled from a ``ModelSpec``: embedding, blocks run in the order
of the run list, final norm on the wanted rows, LM head."""

from __future__ import annotations

import os
from typing import Callable, Mapping

import torch

from ..config.spec import ModelSpec
from .base import CacheNeed, CacheView, ParamSpec, StepContext
from .block import Block
from .registry import make


_NVTX = os.environ.get("PSB200_NVTX", "0") == "1"


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = make("embedding", spec.embedding)
        self.blocks = [Block(layer) for layer in spec.layers]
        self.final_norm = make("norm", spec.final_norm)
        self.head = make("head", spec.head)
        self.compute_dtype: torch.dtype | None = None
        self._lazy_products: bool | None = None  # worked out at the first step (see forward)

    # ---- tensors ---------------------------------------------------------
    def named_parts(self):
        yield "embedding", self.embedding
        for i, block in enumerate(self.blocks):
            for name, p in block.named_parts():
                yield f"layers.{i}.{name}", p
        yield "final_norm", self.final_norm
        yield "head", self.head

    def param_table(self) -> dict[str, ParamSpec]:
        """part path -> wanted tensor, in a fixed order (the random-weights mode draws in this order)."""
        table: dict[str, ParamSpec] = {}
        for prefix, p in self.named_parts():
            for local, ps in p.param_specs().items():
                table[f"{prefix}.{local}"] = ps
        return table

    def load(self, tensors: Mapping[str, torch.Tensor], *, compute_dtype: torch.dtype, device: torch.device,
             max_positions: int) -> None:
        for prefix, p in self.named_parts():
            mine = {local: tensors[f"{prefix}.{local}"] for local in p.param_specs()}
            p.load(mine, compute_dtype=compute_dtype, device=device)
            p.prepare(max_positions=max_positions, compute_dtype=compute_dtype, device=device)
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding.table)
        self.compute_dtype = compute_dtype

    def num_bytes(self) -> int:
        """Bytes of the weights on the device, every tensor once however many parts use it: a tied head is the
        embedding's table (prefixserve/model/weights.py:49-59 counts by data pointer in the same way).  Start-up
        tables that are not in the checkpoint (rotary angles) are not weights and do not count."""
        seen: set[int] = set()
        total = 0
        for _, part in self.named_parts():
            for value in vars(part).values():
                if isinstance(value, torch.Tensor) and value.data_ptr() not in seen:
                    seen.add(value.data_ptr())
                    total += value.numel() * value.element_size()
        return total

    # ---- cache -----------------------------------------------------------
    def cache_needs(self) -> list[CacheNeed]:
        """What each cache entry must hold (entry index -> need of the call that writes it)."""
        needs: list[CacheNeed | None] = [None] * self.spec.num_cache_entries
        for call in self.spec.schedule:
            need = self.blocks[call.layer].mixer.cache_need()
            if call.writes_cache:
                needs[call.cache] = need
        for call in self.spec.schedule:
            if not call.writes_cache:
                need = self.blocks[call.layer].mixer.cache_need()
                if needs[call.cache] != need:
                    raise ValueError(f"layer {call.layer} reads cache entry {call.cache} but needs {need}, entry holds {needs[call.cache]}")
        return [n if n is not None else CacheNeed() for n in needs]

    # ---- one step ----------------------------------------------------------
    def forward(self, ctx: StepContext, cache_view: Callable[[int, bool], CacheView], rows: torch.Tensor) -> torch.Tensor:
        """Runs the step's tokens; returns float32 logits [len(rows), vocab] for the wanted flat rows."""
        if self._lazy_products is None:
            # A sublayer may hand its last product on unrun only if whatever meets it next knows what that is: every
            # block arranged the built-in pre-norm way and every norm saying that it takes one.
            from .block import pre_norm
            norms = [self.final_norm] + [n for b in self.blocks for n in (b.mixer_norm, b.ffn_norm) if n is not None]
            self._lazy_products = (all(b.run is pre_norm for b in self.blocks)
                                   and all(getattr(n, "takes_pending_products", False) for n in norms))
        if self._lazy_products:
            ctx.extras["lazy_products"] = True
        h = self.embedding.forward(ctx.token_ids)
        pending = None
        for at, call in enumerate(self.spec.schedule):
            if _NVTX:  # PSB200_NVTX=1: a named range per run-list entry for timeline tools
                torch.cuda.nvtx.range_push(f"call {at}: layer {call.layer}")
            h, pending = self.blocks[call.layer].forward(h, pending, ctx, cache_view(call.cache, call.writes_cache))
            if _NVTX:
                torch.cuda.nvtx.range_pop()
        if rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=h.device)
        if self.head.takes_deferred_input:
            return self.head.forward(self.final_norm.defer(h, pending, ctx, rows=rows))
        return self.head.forward(self.final_norm.forward(h, pending, ctx, rows=rows))


def build_model(spec: ModelSpec) -> DecoderModel:
    return DecoderModel(spec)
