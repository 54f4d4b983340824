"""The arrangement of parts in a layer.

``PreNormBlock`` (crates/synaptix-models/llm/common/src/model.rs:1179-1199):
``h += mixer(norm1(h)); h += ffn(norm2(h))``.  The residual stream ``h`` is
float32; each branch output is handed on as ``pending`` and added by the next
norm's kernel, so a sum and a norm are one pass over memory.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from .base import FeedForward, Mixer, Norm, Part, PendingLinear, PendingNorm, ScaledRows, StepContext


class PreNormBlock(Part):
    takes_pending_product = True   # forward's ``pending`` may be a PendingLinear

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward):
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn

    def children(self) -> List[Part]:
        return [self.norm1, self.mixer, self.norm2, self.ffn]

    def cache_request(self):
        return self.mixer.cache_request()

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache_view, write_cache: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
        """``pending`` and the second result may be a ``PendingLinear``: a branch's last product handed on unrun,
        so that the norm after it can let it add itself into ``h`` (only between parts that say they can)."""
        if isinstance(pending, PendingLinear) and not self.norm1.takes_pending_product:
            pending = pending.materialize()
        x = self.norm1.add_forward(h, pending, lazy=self.mixer.accepts_lazy_input)
        if self.mixer.can_defer_output and self.norm2.takes_pending_product:
            a = self.mixer.forward(x, ctx, cache_view, write_cache, defer_output=True)
        else:
            a = self.mixer.forward(x, ctx, cache_view, write_cache)
        if isinstance(x, (PendingNorm, ScaledRows)):
            h = x.h_after()
        y = self.norm2.add_forward(h, a, lazy=self.ffn.accepts_lazy_input)
        m = self.ffn.forward(y, ctx, defer_output=True) if self.ffn.can_defer_output else self.ffn.forward(y, ctx)
        if isinstance(y, (PendingNorm, ScaledRows)):
            h = y.h_after()
        return h, m
