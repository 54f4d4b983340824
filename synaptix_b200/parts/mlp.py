"""Dense gated feed-forward (SwiGLU): ``down( silu(x Wg^T) * (x Wu^T) )``,
``silu(x) = x / (1 + exp(-x))`` (crates/synaptix-models/llm/common/src/model.rs:1670-1691;
crates/synaptix-kernels-cuda/src/cu/fused/mlp/silu_and_mul.cu:11-25).  Gate and up
run as one product; the activation is computed in 32-bit.
"""
from __future__ import annotations

from typing import List

import torch

from .base import FeedForward, Part, StepContext
from .linear import Linear


class SwiGLU(FeedForward):
    accepts_lazy_input = True      # x goes straight into the fused gate/up product
    can_defer_output = True        # the down projection may be handed on unrun

    def __init__(self, prefix: str, width: int, intermediate: int):
        self.width, self.intermediate = width, intermediate
        self.gate_up = Linear([prefix + "gate_proj.weight", prefix + "up_proj.weight"], width,
                              [intermediate, intermediate])
        self.down = Linear(prefix + "down_proj.weight", intermediate, width)

    def children(self) -> List[Part]:
        return [self.gate_up, self.down]

    def forward(self, x: torch.Tensor, ctx: StepContext, defer_output: bool = False) -> torch.Tensor:
        z = self.gate_up.forward(x, epilogue="silu_mul")
        return self.down.deferred(z) if defer_output else self.down.forward(z)
