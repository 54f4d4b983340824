"""Grouped-query attention over the paged cache: the mixer of the Qwen3 dense decoder.

In the reference's order (crates/synaptix-models/llm/common/src/model.rs:1715-1734,
1781-1782, 1872-1878):
``q,k,v = x Wq^T, x Wk^T, x Wv^T`` -> per-head RMSNorm of q and k (optional) ->
rotation of q and k (optional) -> k, v appended to the cache ->
``softmax(q k^T * scale + causal mask) v`` with query head ``h`` reading kv head
``h // (nh / nkv)`` -> ``Wo``.  Key ``j`` is visible to the query at position ``p``
iff ``j <= p`` and, with a window ``w``, ``j > p - w``.

Sizes and constants are parameters: heads, kv heads, head size, norm eps, scale,
window, the position encoding.  The three projections run as one product.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch

from .. import ops
from ..cache.store import KVRequest, KVView
from ..weights.loader import TensorSpec
from .base import Mixer, Part, PositionEncoding, Runtime, StepContext, to_device_f32
from .linear import Linear


class Attention(Mixer):
    accepts_lazy_input = True      # x goes straight into the fused q/k/v product
    can_defer_output = True        # the output projection may be handed on unrun

    def __init__(self, prefix: str, width: int, n_heads: int, n_kv_heads: int, head_dim: int, *,
                 position: PositionEncoding, qk_norm_eps: Optional[float] = None,
                 window: Optional[int] = None, scale: Optional[float] = None):
        if n_heads % n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        self.prefix = prefix
        self.width = width
        self.nh, self.nkv, self.hd = n_heads, n_kv_heads, head_dim
        self.position = position
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.qkv = Linear([prefix + "q_proj.weight", prefix + "k_proj.weight", prefix + "v_proj.weight"],
                          width, [n_heads * head_dim, n_kv_heads * head_dim, n_kv_heads * head_dim])
        self.o = Linear(prefix + "o_proj.weight", n_heads * head_dim, width)
        self.wq: Optional[torch.Tensor] = None
        self.wk: Optional[torch.Tensor] = None

    def children(self) -> List[Part]:
        return [self.qkv, self.o, self.position]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        if self.qk_norm_eps is None:
            return {}
        return {self.prefix + "q_norm.weight": TensorSpec((self.hd,), "gain"),
                self.prefix + "k_norm.weight": TensorSpec((self.hd,), "gain")}

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        if self.qk_norm_eps is not None:
            self.wq = to_device_f32(tensors[self.prefix + "q_norm.weight"], rt)
            self.wk = to_device_f32(tensors[self.prefix + "k_norm.weight"], rt)

    def cache_request(self):
        return KVRequest(self.nkv, self.hd, self.window)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache_view: KVView, write_cache: bool = True,
                defer_output: bool = False) -> torch.Tensor:
        out = self.o.deferred if defer_output else self.o.forward
        T = x.shape[0]
        rot = self.position.rotation()
        inv_freq, rotary_dim = rot if rot is not None else (None, 0)
        bt = ctx.block_tables[cache_view.group]
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        if (isinstance(x, torch.Tensor)
                and ops.projection_prepares_heads(T, x.shape[1], x.dtype, self.qkv.weight.dtype, self.nh, self.nkv, self.hd,
                                                  rotary_dim)
                and not ctx.all_single):
            # prompt steps: the projection's epilogue prepares the heads and writes the cache
            q = ops.project_and_prepare(x, self.qkv.weight, cache_view.k if write_cache else None,
                                        cache_view.v if write_cache else None, self.wq, self.wk, inv_freq, eps, ctx, bt,
                                        self.nh, self.nkv, self.hd)
            return out(ops.attention(q, cache_view.k, cache_view.v, ctx, bt, self.nh, self.nkv, self.hd, self.scale, self.window))
        qkv = self.qkv.forward(x)
        if ops.decode_attention_takes_projection(qkv.dtype, self.nh, self.nkv, self.hd, rotary_dim, ctx):
            # single-token steps: the attention kernel prepares the heads and writes the cache itself
            a = ops.attention_from_projection(qkv, cache_view.k, cache_view.v, ctx, bt, self.nh, self.nkv, self.hd,
                                              self.scale, self.window, self.wq, self.wk, inv_freq,
                                              self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, write_cache)
            return out(a)
        q = torch.empty((T, self.nh * self.hd), dtype=qkv.dtype, device=qkv.device)
        ops.qkv_prepare(qkv, q, cache_view.k if write_cache else None, cache_view.v if write_cache else None,
                        self.wq, self.wk, inv_freq, rotary_dim,
                        self.qk_norm_eps if self.qk_norm_eps is not None else 0.0,
                        ctx.positions, ctx.seq_of_token, bt, self.nh, self.nkv, self.hd,
                        pages_like=cache_view.k)
        a = ops.attention(q, cache_view.k, cache_view.v, ctx, bt, self.nh, self.nkv, self.hd,
                          self.scale, self.window)
        return out(a)
