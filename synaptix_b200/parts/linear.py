"""Matrix products ``y = x W^T`` with weight ``[out, in]`` and no bias
(crates/synaptix-nn/src/linear.rs:10-35; the Qwen3 decoder binds every projection
without bias, crates/synaptix-models/llm/common/src/weights.rs:49-51).

``Linear`` may bind several named matrices and stack them along the output
dimension, so that q/k/v (or gate/up) become one product; the checkpoint keeps
its separate tensors and names.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional, Sequence

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Part, PendingLinear, PendingNorm, Runtime, ScaledRows, to_device_matrix


class Linear(Part):
    def __init__(self, weight_names: Sequence[str], in_features: int, out_features: Sequence[int],
                 kind: str = "matrix"):
        if isinstance(weight_names, str):
            weight_names = [weight_names]
            out_features = [out_features]
        self.weight_names = list(weight_names)
        self.in_features = in_features
        self.out_features = list(out_features)
        self.kind = kind
        self.weight: Optional[torch.Tensor] = None

    @property
    def total_out(self) -> int:
        return sum(self.out_features)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {n: TensorSpec((o, self.in_features), self.kind)
                for n, o in zip(self.weight_names, self.out_features)}

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        ws = [to_device_matrix(tensors[n], rt) for n in self.weight_names]
        self.weight = ws[0] if len(ws) == 1 else torch.cat(ws, dim=0).contiguous()

    def share(self, weight: torch.Tensor) -> None:
        """Use an already bound matrix (a tied output head uses the embedding table)."""
        self.weight = weight

    def deferred(self, x: torch.Tensor) -> PendingLinear:
        """This product, not run yet (see ``PendingLinear``)."""
        return PendingLinear(x, self.weight)

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                epilogue: Optional[str] = None) -> torch.Tensor:
        if isinstance(x, ScaledRows):
            y = ops.linear_scaled(x.x, x.ssq, x.eps, self.weight, out_dtype=out_dtype, epilogue=epilogue)
            if y is not None:
                return y
            x = x.materialize()
        if isinstance(x, PendingNorm):
            y = ops.linear_normed(x, self.weight, out_dtype=out_dtype, epilogue=epilogue)
            if y is not None:
                return y
            x = x.materialize()
        return ops.linear(x, self.weight, out_dtype=out_dtype, epilogue=epilogue)
