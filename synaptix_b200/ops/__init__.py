"""The operations of a decoder step, each a hand-written CUDA kernel for sm_100a.

This layer chooses, for the sizes and dtype at hand, between the fast kernel of an
operation and the plain one that takes every size (``ops.generic``).  There is no
CPU path and no library fallback: without a CUDA device or without ``nvcc`` to build
the kernels, every call raises ``KernelsUnavailable``.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc.build import KernelsUnavailable
from ._lib import KernelError, set_launch_counter
from .generic import (add_rmsnorm, attn_generic, decode_advance, embed_gather, gemm_generic, qkv_prepare,
                      residual_add,
                      silu_mul)

__all__ = ["KernelsUnavailable", "KernelError", "set_launch_counter", "decode_advance", "add_rmsnorm", "attn_generic", "embed_gather",
           "gemm_generic", "qkv_prepare", "residual_add", "silu_mul", "linear", "attention"]


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x[M, K] @ w[N, K].T`` with 32-bit accumulation; output in ``out_dtype`` (default ``x``'s)."""
    return gemm_generic(x, w, out_dtype=out_dtype)


def attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, ctx, block_table: torch.Tensor,
              nh: int, nkv: int, hd: int, scale: float, window: Optional[int]) -> torch.Tensor:
    """Causal attention of the step's packed queries over the cache (which already holds
    this step's keys and values)."""
    return attn_generic(q, k_pages, v_pages, ctx.positions, ctx.seq_of_token, block_table, nh, nkv, hd,
                        scale, window)
