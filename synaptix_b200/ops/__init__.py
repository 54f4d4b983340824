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
from .attention import (TC_TILE_ROWS, attn_decode, attn_decode_prep, attn_decode_tma, attn_prefill, attn_prefill_tc,
                        fast_supported, pick_splits, query_tiles, tc_prefill_supported, tma_decode_supported)
from .decode import MAX_ROWS as SKINNY_MAX_ROWS, skinny_gemm, skinny_gemm_residual, skinny_gemm_scaled, skinny_supported
from .gemm_tc import gemm_tc, gemm_tc_qkv, qkv_epilogue_supported, tc_supported
from .gemm_ws import gemm_ws, gemm_ws_residual, ws_supported
from .options import OPTIONS, KernelOptions, options, set_options
from .generic import (add_rmsnorm, attn_generic, decode_advance, decode_begin, embed_gather, gemm_generic, qkv_prepare,
                      residual_add, rope_table, silu_mul)

__all__ = ["OPTIONS", "KernelOptions", "options", "set_options", "KernelsUnavailable", "KernelError", "set_launch_counter", "decode_advance", "decode_begin", "check_status", "add_rmsnorm", "attn_generic", "embed_gather",
           "gemm_generic", "qkv_prepare", "residual_add", "silu_mul", "linear", "linear_normed", "norm_fusable", "attention",
           "attention_from_projection", "decode_attention_takes_projection", "residual_product_fusable",
           "linear_into_residual", "linear_scaled", "projection_prepares_heads", "project_and_prepare", "rope_table"]


_STATUS_READERS = {"gemm_tc": ("the tcgen05 matrix product (gemm_tc)", "gemm_tc_status"),
                   "attn_tc": ("the tcgen05 prompt attention (attn_tc)", "attn_tc_status"),
                   "attn_decode": ("the TMA-fed decode attention (attn_decode)", "attn_decode_status"),
                   "gemm_ws": ("the weight-streaming tcgen05 product (gemm_ws)", "gemm_ws_status")}


def check_status(readers=None) -> None:
    """Raise ``KernelError`` if a bounded wait inside a tensor-memory kernel ran out in a launch the host has
    since waited for: that kernel returned without writing (all of) its output.  The status word is put back to
    0 (and the product's cut-tile counters are zeroed) so that later launches start clean.  Libraries that were
    never loaded have launched nothing and are not looked at; reading costs no device call.

    ``readers``: ``{name: (description, function(reset) -> code)}`` to look at instead (tests)."""
    if readers is None:
        from ._lib import loaded
        from .attention import attn_decode_status, attn_tc_status
        from .gemm_tc import gemm_tc_status
        from .gemm_ws import gemm_ws_status
        fns = {"gemm_tc_status": gemm_tc_status, "attn_tc_status": attn_tc_status, "attn_decode_status": attn_decode_status,
               "gemm_ws_status": gemm_ws_status}
        readers = {}
        for lib, (what, fname) in _STATUS_READERS.items():
            if loaded(lib):
                readers[lib] = (what, fns[fname])
    for lib, (what, read) in readers.items():
        code = read(False)
        if code:
            read(True)
            raise KernelError(f"{what}: a bounded wait inside the kernel ran out (status {code}); "
                              "its output is incomplete and the step's results must not be used")


# The weight-streaming tcgen05 product takes up to 256 rows; the step function gives it up to this many.  Measured at
# Qwen3-4B sizes, us for q/k/v + o + gate/up + down in replayed graphs: 144 rows 90 against 100 with the tile product of
# prompt steps, 192 rows 109 against 101, 256 rows 124 against 103 (one block of 256 rows of partial results fills an
# SM's shared memory, and the 152 tiles of gate/up then take 62 us).
WS_MAX_ROWS = 160

# The weight-streaming product of 17 to 160 rows makes one block per 128 outputs; an output head has a thousand of
# them, and there the persistent product with its 256-wide tiles measured faster (142 against 158 us for 151,936
# outputs of 64 rows).
WS_MAX_OUT = 32768

# Up to 16 rows both weight-streaming products apply.  The tcgen05 one streams faster and has the longer beginning and
# end, so it takes the matrices of 15 M elements and more (at 8 rows and Qwen3-4B sizes, us in replayed graphs: gate/up
# 19.3 against 22.8, down 12.2 against 13.9, q/k/v 8.0 against 8.4) and everything at 9 to 16 rows, where the
# mma.sync kernel needs a second tile of rows (a layer's four products at 16 rows: 47 against 77 us).  The 10 M
# elements of the o product are faster there too when timed alone (6.7 against 6.8) but slower in a step, behind the
# attention kernel (2,874 against 2,944 tok/s at batch 8).
WS_FEW_ROWS_MIN_ELEMENTS = 15_000_000

# A step of ONE row norms inside the next product's prologue (every block repeats the norm of the row) and keeps the
# mma.sync kernels throughout; from two rows on the o / down product adds itself into the residual stream and the next
# product applies the rows' factors (batch 2: 934 against 907 tok/s; batch 1: 492 against 506).
PROLOGUE_NORM_MAX_ROWS = 1


_STREAM_KERNEL = {}


def _weight_stream_kernel(M: int, N: int, K: int, x_dtype, w_dtype) -> Optional[str]:
    """Which weight-streaming product takes ``M <= 160`` rows against ``w[N, K]``: ``"skinny"`` (mma.sync, up to 16
    rows), ``"ws"`` (tcgen05, up to 160 rows and 32,768 outputs) or ``None``.  (Remembered per shape: a step asks
    several times per product, and a prompt step of a few dozen tokens is bound by the host.)"""
    key = (M, N, K, x_dtype, w_dtype, OPTIONS.gemm_ws)
    kind = _STREAM_KERNEL.get(key, 0)
    if kind == 0:
        kind = _STREAM_KERNEL[key] = _pick_weight_stream_kernel(M, N, K, x_dtype, w_dtype)
    return kind


def _pick_weight_stream_kernel(M: int, N: int, K: int, x_dtype, w_dtype) -> Optional[str]:
    skinny = skinny_supported(M, N, K, x_dtype, w_dtype)
    ws = OPTIONS.gemm_ws and N <= WS_MAX_OUT and M <= WS_MAX_ROWS and ws_supported(M, N, K, x_dtype, w_dtype)
    if skinny and ws:
        if M <= PROLOGUE_NORM_MAX_ROWS:          # (one row: batch 1 measured 506 tok/s with mma.sync throughout, 494 with tcgen05 for down)
            return "skinny"
        return "ws" if (M > 8 or N * K >= WS_FEW_ROWS_MIN_ELEMENTS) else "skinny"
    return "skinny" if skinny else ("ws" if ws else None)


# Every block of a product that applies row factors fetches the partial sums; an output head has thousands of
# blocks, and there one norm kernel before it is cheaper (132 against 122 us for 151,936 outputs of 8 rows).
SCALED_MAX_OUT = 65536


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           epilogue: Optional[str] = None) -> torch.Tensor:
    """``x[M, K] @ w[N, K].T`` with 32-bit accumulation; output in ``out_dtype`` (default ``x``'s).
    ``epilogue="silu_mul"``: ``w`` is ``[gate; up]`` stacked and the result is
    ``silu(x gate^T) * (x up^T)``, ``[M, N/2]``."""
    M, K = x.shape
    N = w.shape[0]
    if out_dtype is None:
        out_dtype = x.dtype
    # up to 160 rows: stream W once (mma.sync or tcgen05 with W as the M side, see _weight_stream_kernel); more: the
    # tcgen05 product of prompt steps
    stream_k = _weight_stream_kernel(M, N, K, x.dtype, w.dtype) if out_dtype in (torch.bfloat16, torch.float32) else None
    if stream_k is not None:
        product = skinny_gemm if stream_k == "skinny" else gemm_ws
        if epilogue == "silu_mul":
            if out_dtype == torch.bfloat16:
                return product(x, w, epilogue="silu_mul")
        else:
            return product(x, w, epilogue="f32" if out_dtype == torch.float32 else None)
    if tc_supported(M, N, K, x.dtype, w.dtype) and out_dtype in (torch.bfloat16, torch.float32):
        if epilogue == "silu_mul":
            if out_dtype == torch.bfloat16:
                return gemm_tc(x, w, epilogue="silu_mul")
        else:
            return gemm_tc(x, w, epilogue="f32" if out_dtype == torch.float32 else None)
    y = gemm_generic(x, w, out_dtype=out_dtype if epilogue is None else x.dtype)
    if epilogue == "silu_mul":
        y = silu_mul(y)
    return y


def norm_fusable(M: int, K: int, dtype) -> bool:
    """Can ``rmsnorm(h + delta)`` of ``M`` rows of width ``K`` run inside the next product's prologue?"""
    # every block repeats the norm, so it pays only while the rows are few
    return dtype == torch.bfloat16 and 0 < M <= PROLOGUE_NORM_MAX_ROWS and K % 32 == 0 and K <= 4096


def linear_normed(pn, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                  epilogue: Optional[str] = None) -> Optional[torch.Tensor]:
    """``rmsnorm(pn.h + pn.delta) * gain @ w.T`` in one kernel, or ``None`` if that cannot be fused."""
    M, K = pn.h.shape
    if out_dtype is None:
        out_dtype = pn.dtype
    if not (norm_fusable(M, K, pn.dtype) and w.dtype == torch.bfloat16 and w.shape[1] == K):
        return None
    if epilogue == "silu_mul":
        if out_dtype != torch.bfloat16:
            return None
        epi = "silu_mul"
    elif epilogue is None and out_dtype in (torch.bfloat16, torch.float32):
        epi = "f32" if out_dtype == torch.float32 else None
    else:
        return None
    return skinny_gemm(None, w, epilogue=epi, norm_h=pn.h, norm_delta=pn.delta, norm_h_out=pn.h_out(),
                       norm_gain=pn.gain, norm_eps=pn.eps)


def residual_product_fusable(M: int, N: int, K: int, dtype) -> bool:
    """Can the product ``x[M, K] @ w[N, K].T`` add itself into the residual stream and prepare the norm after the
    sum (``linear_into_residual``)?  2 to 160 rows in bfloat16 (option ``fused_residual``)."""
    # one row: the norm in the consumer's prologue (norm_fusable) measured faster (506 against 492 tok/s)
    if dtype != torch.bfloat16 or not OPTIONS.fused_residual or K <= 0 or M <= PROLOGUE_NORM_MAX_ROWS:
        return False
    return _weight_stream_kernel(M, N, K, dtype, dtype) is not None


def linear_into_residual(x: torch.Tensor, w: torch.Tensor, h: torch.Tensor, gain: torch.Tensor):
    """``h += x @ w.T`` (float32, in place); returns ``(bf16(h * gain), ssq)``: the rows of the RMSNorm after the
    sum without their factor ``rsqrt(mean(h^2) + eps)``, and partial sums of squares of ``h`` from which
    ``linear_scaled`` forms that factor."""
    if _weight_stream_kernel(x.shape[0], w.shape[0], w.shape[1], x.dtype, w.dtype) == "skinny":
        return skinny_gemm_residual(x, w, h, gain)
    return gemm_ws_residual(x, w, h, gain)


def linear_scaled(x: torch.Tensor, ssq: torch.Tensor, eps: float, w: torch.Tensor,
                  out_dtype: Optional[torch.dtype] = None, epilogue: Optional[str] = None) -> Optional[torch.Tensor]:
    """``(x * rsqrt(sum(ssq) / K + eps)) @ w.T`` with the factor applied to the results; ``None`` if no kernel
    does that for these sizes."""
    M, K = x.shape
    if out_dtype is None:
        out_dtype = x.dtype
    stream_k = _weight_stream_kernel(M, w.shape[0], K, x.dtype, w.dtype)
    if stream_k is None or w.shape[1] != K or w.shape[0] > SCALED_MAX_OUT:
        return None
    if epilogue == "silu_mul":
        if out_dtype != torch.bfloat16:
            return None
        epi = "silu_mul"
    elif epilogue is None and out_dtype in (torch.bfloat16, torch.float32):
        epi = "f32" if out_dtype == torch.float32 else None
    else:
        return None
    if stream_k == "skinny":
        return skinny_gemm_scaled(x, w, ssq, eps, epilogue=epi)
    return gemm_ws(x, w, epilogue=epi, ssq=ssq, eps=eps)


# Fewer rows than this and the fused projection is one of the weight-streaming products, which have no such epilogue.
QKV_EPILOGUE_MIN_ROWS = WS_MAX_ROWS + 1


def projection_prepares_heads(M: int, K: int, x_dtype, w_dtype, nh: int, nkv: int, hd: int, rotary_dim: Optional[int]) -> bool:
    """Can the q/k/v product of a prompt step prepare the heads in its epilogue (``project_and_prepare``)?  (Option
    ``qkv_epilogue``.)"""
    return (OPTIONS.qkv_epilogue and M >= QKV_EPILOGUE_MIN_ROWS and rotary_dim in (None, 0, hd)
            and qkv_epilogue_supported(M, nh, nkv, hd, K, x_dtype, w_dtype))


def project_and_prepare(x: torch.Tensor, w: torch.Tensor, k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                        wq, wk, inv_freq, eps: float, ctx, block_table: torch.Tensor, nh: int, nkv: int, hd: int) -> torch.Tensor:
    """The prepared queries ``[T, nh * hd]`` of a prompt step straight from the block's input: the fused q/k/v product
    with the head preparation (per-head RMSNorm, rotation, cache write) as its epilogue.  The cosines and sines of the
    step's angles are made once a step and rotation (``ctx.scratch``) and shared by the layers."""
    cos = sin = None
    if inv_freq is not None:
        key = ("rope_table", inv_freq.data_ptr())
        table = ctx.scratch.get(key)
        if table is None:
            table = ctx.scratch[key] = rope_table(ctx.positions[:x.shape[0]], inv_freq)
        cos, sin = table
    q = torch.empty((x.shape[0], nh * hd), dtype=x.dtype, device=x.device)
    gemm_tc_qkv(x, w, q, k_pages, v_pages, wq, wk, cos, sin, eps, ctx.positions[:x.shape[0]], ctx.seq_of_token[:x.shape[0]],
                block_table, nh, nkv)
    return q


def decode_attention_takes_projection(dtype, nh: int, nkv: int, hd: int, rotary_dim: Optional[int], ctx) -> bool:
    """Can the attention kernel of a single-token step prepare the heads itself (norm, rotation, cache write) from
    the fused projection?  (Option ``attn_prep``.)"""
    return (fast_supported(dtype, nh, nkv, hd) and rotary_dim in (None, 0, hd) and ctx.all_single
            and OPTIONS.attn_prep)


def attention_from_projection(qkv: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, ctx,
                              block_table: torch.Tensor, nh: int, nkv: int, hd: int, scale: float,
                              window: Optional[int], wq, wk, inv_freq, eps: float, write_cache: bool) -> torch.Tensor:
    """Single-token steps: head preparation and attention in one kernel (see ``attn_decode_prep``)."""
    max_pages = (ctx.max_len + 63) // 64
    if OPTIONS.attn_tma and tma_decode_supported(qkv.dtype, nh, nkv, hd):
        return attn_decode_tma(qkv, k_pages, v_pages, ctx.seq_lens, block_table, nh, nkv, hd, scale, window,
                               pick_splits(ctx.n_seqs, nkv, max_pages, qkv.device), prep=True, wq=wq, wk=wk,
                               inv_freq=inv_freq, eps=eps, write_cache=write_cache)
    return attn_decode_prep(qkv, k_pages, v_pages, ctx.seq_lens, block_table, nh, nkv, hd, scale, window,
                            pick_splits(ctx.n_seqs, nkv, max_pages, qkv.device), wq, wk, inv_freq, eps, write_cache)


def attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, ctx, block_table: torch.Tensor,
              nh: int, nkv: int, hd: int, scale: float, window: Optional[int]) -> torch.Tensor:
    """Causal attention of the step's packed queries over the cache (which already holds
    this step's keys and values)."""
    if fast_supported(q.dtype, nh, nkv, hd):
        if ctx.all_single:
            max_pages = (ctx.max_len + 63) // 64
            if OPTIONS.attn_tma and tma_decode_supported(q.dtype, nh, nkv, hd):
                return attn_decode_tma(q, k_pages, v_pages, ctx.seq_lens, block_table, nh, nkv, hd, scale, window,
                                       pick_splits(ctx.n_seqs, nkv, max_pages, q.device))
            return attn_decode(q, k_pages, v_pages, ctx.seq_lens, block_table, nh, nkv, hd, scale, window,
                               pick_splits(ctx.n_seqs, nkv, max_pages, q.device))
        if ctx.host is not None:
            # prompt steps: tcgen05 kernel (128-row tiles) for head size 128, else the mma.sync kernel (64-row tiles)
            tc = tc_prefill_supported(q.dtype, nh, nkv, hd)
            rows = TC_TILE_ROWS if tc else 64
            tiles = ctx.scratch.get(("query_tiles", rows))
            if tiles is None:
                import numpy as np
                ts, t0 = query_tiles(ctx.host["cu_seqlens"], rows)
                both = torch.from_numpy(np.asarray([ts, t0], dtype=np.int32)).to(q.device, non_blocking=True)
                tiles = ctx.scratch[("query_tiles", rows)] = (both[0], both[1])
            kernel = attn_prefill_tc if tc else attn_prefill
            return kernel(q, k_pages, v_pages, tiles[0], tiles[1], ctx.cu_seqlens, ctx.seq_past, ctx.seq_lens,
                          block_table, nh, nkv, hd, scale, window)
    return attn_generic(q, k_pages, v_pages, ctx.positions, ctx.seq_of_token, block_table, nh, nkv, hd,
                        scale, window)
