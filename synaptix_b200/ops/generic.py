"""Python faces of the plain kernels in ``csrc/generic.cu`` (every size, float32 and bfloat16)."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import (KernelError, c_float, c_int, c_longlong, check, dt_code, fn, ptr, require_cuda,
                   stream)


def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = float32(table[ids[t]])``; ``ids`` int32 ``[T]``; result float32 ``[T, H]``."""
    require_cuda(table, ids, out)
    V, H = table.shape
    T = ids.numel()
    if ids.dtype != torch.int32:
        raise KernelError("token ids must be int32")
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    check(fn("generic", "sx_embed_gather")(ptr(table), c_int(dt_code(table.dtype)), ptr(ids), ptr(out),
                                           c_int(T), c_int(H), c_int(V), stream()), "embed_gather")
    return out


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Residual sum and RMSNorm in one pass.

    ``h`` float32 ``[T, H]`` is the residual stream.  With ``delta`` (same shape,
    ``out_dtype``) ``h += delta`` first (written back unless ``rows`` is given).
    Returns ``rmsnorm(h) * weight`` in ``out_dtype``; with ``rows`` (int32 ``[R]``)
    only for those rows, as ``[R, H]``.
    """
    require_cuda(h, delta, weight, rows, out)
    if h.dtype != torch.float32 or weight.dtype != torch.float32:
        raise KernelError("the residual stream and norm gains are float32")
    T, H = h.shape
    if delta is not None and (delta.dtype != out_dtype or delta.shape != h.shape):
        raise KernelError("delta must have the residual's shape and the output dtype")
    if weight.numel() != H:
        raise KernelError(f"norm gain has {weight.numel()} elements for width {H}")
    R = T if rows is None else rows.numel()
    if out is None:
        out = torch.empty((R, H), dtype=out_dtype, device=h.device)
    check(fn("generic", "sx_add_rmsnorm")(ptr(h), ptr(delta), ptr(weight), c_float(eps), ptr(out), ptr(rows),
                                          c_int(R), c_int(H), c_int(dt_code(out_dtype)),
                                          c_int(1 if rows is None else 0), stream()), "add_rmsnorm")
    return out


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> None:
    """``h += delta`` with ``h`` float32."""
    require_cuda(h, delta)
    if h.dtype != torch.float32 or h.shape != delta.shape:
        raise KernelError("residual_add: h must be float32 and shapes equal")
    check(fn("generic", "sx_residual_add")(ptr(h), ptr(delta), c_longlong(h.numel()),
                                           c_int(dt_code(delta.dtype)), stream()), "residual_add")


def gemm_generic(a: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a[M, K] @ w[N, K].T`` with 32-bit accumulation on CUDA cores (no tensor cores)."""
    require_cuda(a, w, out)
    M, K = a.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: inner sizes differ ({K} and {K2})")
    if out_dtype is None:
        out_dtype = a.dtype
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    check(fn("generic", "sx_gemm_generic")(ptr(a), c_int(dt_code(a.dtype)), ptr(w), c_int(dt_code(w.dtype)),
                                           ptr(out), c_int(dt_code(out.dtype)), c_int(M), c_int(N), c_int(K),
                                           stream()), "gemm_generic")
    return out


def qkv_prepare(qkv: torch.Tensor, q_out: torch.Tensor, k_pages: Optional[torch.Tensor],
                v_pages: Optional[torch.Tensor], wq: Optional[torch.Tensor], wk: Optional[torch.Tensor],
                inv_freq: Optional[torch.Tensor], rotary_dim: int, eps: float, positions: torch.Tensor,
                seq_of_token: torch.Tensor, block_table: torch.Tensor, nh: int, nkv: int, hd: int,
                pages_like: Optional[torch.Tensor] = None) -> None:
    """Per-head RMSNorm (optional), rotate-half rotation (optional) and the cache write.

    ``qkv`` ``[T, (nh + 2 nkv) * hd]``; q heads go to ``q_out`` ``[T, nh * hd]``; k and v
    heads go into the pages ``[n_pages, nkv, 64, hd]`` of the token's sequence at the
    token's position.  With ``k_pages``/``v_pages`` ``None`` nothing is written to the cache
    (a layer that reads another layer's cache).
    """
    require_cuda(qkv, q_out, k_pages, v_pages, wq, wk, inv_freq, positions, seq_of_token, block_table)
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd:
        raise KernelError("qkv_prepare: qkv has the wrong width")
    if qkv.dtype != q_out.dtype:
        raise KernelError("qkv_prepare: qkv and q must share a dtype")
    n_pages = 0
    for pg in (k_pages, v_pages):
        if pg is None:
            continue
        if pg.dtype != qkv.dtype:
            raise KernelError("qkv_prepare: qkv and the cache must share a dtype")
        if pg.dim() != 4 or tuple(pg.shape[1:]) != (nkv, 64, hd):
            raise KernelError("qkv_prepare: cache pages must be [n_pages, nkv, 64, hd]")
        n_pages = pg.shape[0]
    for t in (positions, seq_of_token, block_table):
        if t.dtype != torch.int32:
            raise KernelError("qkv_prepare: index tensors are int32")
    check(fn("generic", "sx_qkv_prepare")(
        ptr(qkv), ptr(q_out), ptr(k_pages), ptr(v_pages), ptr(wq), ptr(wk), ptr(inv_freq), c_int(rotary_dim),
        c_float(eps), ptr(positions), ptr(seq_of_token), ptr(block_table), c_int(block_table.shape[1]),
        c_int(T), c_int(nh), c_int(nkv), c_int(hd), c_int(n_pages), c_int(dt_code(qkv.dtype)),
        stream()), "qkv_prepare")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor):
    """``(cos, sin)`` float32 ``[T, pairs]`` of ``position * inv_freq[i]`` (32-bit angles, ``sincosf``)."""
    require_cuda(positions, inv_freq)
    T, pairs = positions.numel(), inv_freq.numel()
    cs = torch.empty((T, pairs), dtype=torch.float32, device=positions.device)
    sn = torch.empty_like(cs)
    check(fn("generic", "sx_rope_table")(ptr(positions), ptr(inv_freq), c_int(pairs), c_int(T), ptr(cs), ptr(sn), stream()),
          "rope_table")
    return cs, sn


def attn_generic(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, positions: torch.Tensor,
                 seq_of_token: torch.Tensor, block_table: torch.Tensor, nh: int, nkv: int, hd: int,
                 scale: float, window: Optional[int] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal (optionally windowed) attention of packed tokens over the paged cache, 32-bit math."""
    require_cuda(q, k_pages, v_pages, positions, seq_of_token, block_table, out)
    T = q.shape[0]
    if out is None:
        out = torch.empty((T, nh * hd), dtype=q.dtype, device=q.device)
    check(fn("generic", "sx_attn_generic")(
        ptr(q), ptr(k_pages), ptr(v_pages), ptr(out), ptr(positions), ptr(seq_of_token), ptr(block_table),
        c_int(block_table.shape[1]), c_int(T), c_int(nh), c_int(nkv), c_int(hd), c_float(scale),
        c_int(0 if window is None else int(window)), c_int(dt_code(q.dtype)), stream()), "attn_generic")
    return out


def silu_mul(gu: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(gu[:, :I]) * gu[:, I:]`` for ``gu`` ``[T, 2I]``."""
    require_cuda(gu, out)
    T, I2 = gu.shape
    I = I2 // 2
    if out is None:
        out = torch.empty((T, I), dtype=gu.dtype, device=gu.device)
    check(fn("generic", "sx_silu_mul")(ptr(gu), ptr(out), c_int(T), c_int(I), c_int(dt_code(gu.dtype)), stream()),
          "silu_mul")
    return out


def decode_begin(token_ids: torch.Tensor, control: torch.Tensor, history: Optional[torch.Tensor] = None,
                 hist_len: Optional[torch.Tensor] = None) -> None:
    """On the device, before a decode step: ``token_ids[i] = control[i]`` where ``control[i] >= 0``
    (and the last entry of row ``i``'s history becomes that token)."""
    require_cuda(token_ids, control, history, hist_len)
    check(fn("generic", "sx_decode_begin")(ptr(token_ids), ptr(control), ptr(history), ptr(hist_len),
                                           c_int(0 if history is None else history.shape[1]),
                                           c_int(token_ids.numel()), stream()), "decode_begin")


def decode_advance(token_ids: torch.Tensor, sampled: torch.Tensor, positions: torch.Tensor,
                   seq_past: torch.Tensor, seq_lens: torch.Tensor, rng_step: Optional[torch.Tensor] = None,
                   advance_by: Optional[torch.Tensor] = None, history: Optional[torch.Tensor] = None,
                   hist_len: Optional[torch.Tensor] = None) -> None:
    """On the device, after a decode step: for every row with ``advance_by[i] != 0`` (all rows if absent)
    ``token_ids = sampled``, position, lengths and ``rng_step`` grow by one, and the sampled token is
    appended to the row's ``history [S, cap]`` (``hist_len`` grows)."""
    require_cuda(token_ids, sampled, positions, seq_past, seq_lens, rng_step, advance_by, history, hist_len)
    check(fn("generic", "sx_decode_advance")(ptr(token_ids), ptr(sampled), ptr(positions), ptr(seq_past),
                                             ptr(seq_lens), ptr(rng_step), ptr(advance_by), ptr(history),
                                             ptr(hist_len), c_int(0 if history is None else history.shape[1]),
                                             c_int(token_ids.numel()), stream()), "decode_advance")
