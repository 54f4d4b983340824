"""Token embedding and the output head.

``h0[t] = E[id_t]`` with no scale (crates/synaptix-ops/src/embed/token_embed.rs:4-15);
logits ``= norm(h)[rows] W^T`` with ``W = E`` when tied
(crates/synaptix-models/llm/common/src/model.rs:757-772,1068-1094), computed only for
the rows asked for and returned in float32.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Part, Runtime, to_device_matrix
from .linear import Linear


class Embedding(Part):
    def __init__(self, weight_name: str, vocab: int, width: int):
        self.weight_name, self.vocab, self.width = weight_name, vocab, width
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.vocab, self.width), "embedding")}

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.weight = to_device_matrix(tensors[self.weight_name], rt)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        """float32 residual stream ``[T, width]``."""
        return ops.embed_gather(self.weight, token_ids)


class OutputHead(Part):
    """``tied`` is True, False, or None (= tied iff the weights hold no matrix of that name)."""

    def __init__(self, weight_name: str, vocab: int, width: int, tied: Optional[bool], embedding: Embedding):
        self.weight_name, self.vocab, self.width = weight_name, vocab, width
        self.tied = tied
        self.embedding = embedding
        self.linear = Linear(weight_name, width, vocab)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        # a tied checkpoint may still carry a copy of the matrix; it is then ignored
        return {self.weight_name: TensorSpec((self.vocab, self.width), "matrix", optional=self.tied is not False)}

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        tied = self.tied if self.tied is not None else (self.weight_name not in tensors)
        if tied:
            self.linear.share(self.embedding.weight)
        else:
            self.linear.bind(tensors, rt)
        self.is_tied = tied

    def forward(self, x) -> torch.Tensor:
        """``x``: the normalised rows, or a ``PendingNorm`` of them."""
        return self.linear.forward(x, out_dtype=torch.float32)
