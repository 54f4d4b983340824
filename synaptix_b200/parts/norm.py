"""RMSNorm with a plain gain, fused with the residual sum.

Formula (crates/synaptix-ops/src/norm/rms_norm.rs:17-26; CUDA
crates/synaptix-kernels-cuda/src/cu/reduction/rms_norm.cu:84-96):
``y = x * rsqrt(mean(x^2) + eps) * w`` in 32-bit, gain ``w`` (not ``1 + w``).
The residual stream itself is float32 here, so the sum ``h + delta`` is never
rounded to the compute dtype (the reference rounds it, rmsnorm_residual.cu:97-159).
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Norm, PendingLinear, PendingNorm, Runtime, ScaledRows, to_device_f32


class RMSNorm(Norm):
    def __init__(self, weight_name: str, width: int, eps: float):
        self.weight_name = weight_name
        self.width = width
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None
        self._dtype = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.width,), "gain")}

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.weight = to_device_f32(tensors[self.weight_name], rt)
        self._dtype = rt.dtype

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return ops.add_rmsnorm(h, None, self.weight, self.eps, self._dtype)

    takes_pending_product = True

    def add_forward(self, h, delta, rows=None, lazy=False):
        if isinstance(delta, PendingLinear):
            N, K = delta.weight.shape
            if (lazy and rows is None and N == self.width and h.dtype == torch.float32 and h.is_contiguous()
                    and delta.weight.dtype == self._dtype and delta.x.dtype == self._dtype
                    and ops.residual_product_fusable(h.shape[0], N, K, self._dtype)):
                # the product adds itself into h and leaves the rows of this norm without their factor
                x, ssq = ops.linear_into_residual(delta.x, delta.weight, h, self.weight)
                return ScaledRows(x, ssq, self.eps, h, self.weight, self._dtype)
            delta = delta.materialize()
        if lazy and rows is None and ops.norm_fusable(h.shape[0], h.shape[1], self._dtype):
            return PendingNorm(h, delta, self.weight, self.eps, self._dtype)
        return ops.add_rmsnorm(h, delta, self.weight, self.eps, self._dtype, rows=rows)
