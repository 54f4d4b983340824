"""Python face of the weight-streaming products in ``csrc/decode.cu`` (bfloat16, up to 16 rows)."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import KernelError, c_float, c_int, check, fn, ptr, require_cuda, stream

_EPI = {None: 0, "f32": 1, "silu_mul": 2}
MAX_ROWS = 16          # more rows go to the tcgen05 product, which takes every K this kernel takes


def skinny_supported(M: int, N: int, K: int, x_dtype, w_dtype) -> bool:
    return (x_dtype == torch.bfloat16 and w_dtype == torch.bfloat16 and 0 < M <= MAX_ROWS and K % 32 == 0 and K > 0)


def pick_ks(tiles: int, K: int = 0) -> int:
    """Warps of a block that split K.  8 everywhere (measured best on a B200), except 16 (blocks of
    16 warps) for matrices with so few row tiles that 8 warps a tile leave the SMs short of warps."""
    if tiles <= 192 and K >= 2048:
        return 16
    return 8


def skinny_gemm(x: Optional[torch.Tensor], w: torch.Tensor, *, epilogue: Optional[str] = None,
                ks: Optional[int] = None, out: Optional[torch.Tensor] = None,
                norm_h: Optional[torch.Tensor] = None, norm_delta: Optional[torch.Tensor] = None,
                norm_h_out: Optional[torch.Tensor] = None, norm_gain: Optional[torch.Tensor] = None,
                norm_eps: float = 0.0) -> torch.Tensor:
    """``x[M, K] @ w[N, K].T`` for ``M <= 16`` rows, reading ``w`` once (``ks``: 8 or 16 warps split K).

    ``epilogue``: ``None`` -> bfloat16 ``[M, N]``; ``"f32"`` -> float32 ``[M, N]``;
    ``"silu_mul"`` -> ``w`` is ``[gate; up]`` stacked, result bfloat16 ``[M, N/2]``.
    With ``norm_h`` (float32 ``[M, K]``) the activations are computed inside the kernel as
    ``rmsnorm(norm_h + norm_delta) * norm_gain`` and ``norm_h + norm_delta`` is written to
    ``norm_h_out`` (which must not alias ``norm_h``); then ``M <= 2`` and ``x`` is ``None``.
    """
    require_cuda(x, w, out, norm_h, norm_delta, norm_h_out, norm_gain)
    N, K = w.shape
    M = (x if x is not None else norm_h).shape[0]
    if (x if x is not None else norm_h).shape[1] != K:
        raise KernelError("skinny_gemm: inner sizes differ")
    if epilogue not in _EPI:
        raise KernelError(f"skinny_gemm: unknown epilogue {epilogue!r}")
    if norm_h is not None:
        if norm_h.dtype != torch.float32 or norm_gain is None or norm_gain.dtype != torch.float32:
            raise KernelError("skinny_gemm: the norm prologue takes float32 h and gain")
        if norm_h_out is not None and norm_h_out.data_ptr() == norm_h.data_ptr():
            raise KernelError("skinny_gemm: norm_h_out must not alias norm_h")
    n_out = N // 2 if epilogue == "silu_mul" else N
    if out is None:
        out = torch.empty((M, n_out), dtype=torch.float32 if epilogue == "f32" else torch.bfloat16, device=w.device)
    tiles = (n_out + 7) // 8 if epilogue == "silu_mul" else (N + 15) // 16
    if ks is None:
        ks = pick_ks(tiles, K)
    check(fn("decode", "sx_skinny_gemm")(ptr(x), ptr(w), ptr(out), c_int(M), c_int(N), c_int(K), c_int(_EPI[epilogue]),
                                         c_int(ks), ptr(norm_h), ptr(norm_delta), ptr(norm_h_out), ptr(norm_gain),
                                         c_float(norm_eps), stream()), "skinny_gemm")
    return out


def skinny_gemm_scaled(x: torch.Tensor, w: torch.Tensor, ssq: Optional[torch.Tensor], eps: float, *,
                       epilogue: Optional[str] = None, ks: Optional[int] = None) -> torch.Tensor:
    """``skinny_gemm`` for rows of ``x`` that lack their RMSNorm factor: row ``b`` of the result is multiplied by
    ``rsqrt(sum(ssq[b]) / K + eps)`` (``ssq`` float32 ``[M, n]``: partial sums of squares of the row the norm is of)."""
    require_cuda(x, w, ssq)
    N, K = w.shape
    M = x.shape[0]
    if x.shape[1] != K or epilogue not in _EPI:
        raise KernelError("skinny_gemm_scaled: inner sizes differ or unknown epilogue")
    if ssq is not None and (ssq.dtype != torch.float32 or ssq.shape[0] != M or not ssq.is_contiguous()):
        raise KernelError("skinny_gemm_scaled: ssq must be contiguous float32 [M, n]")
    n_out = N // 2 if epilogue == "silu_mul" else N
    out = torch.empty((M, n_out), dtype=torch.float32 if epilogue == "f32" else torch.bfloat16, device=w.device)
    tiles = (n_out + 7) // 8 if epilogue == "silu_mul" else (N + 15) // 16
    if ks is None:
        ks = pick_ks(tiles, K)
    check(fn("decode", "sx_skinny_gemm_norm")(
        ptr(x), ptr(w), ptr(out), c_int(M), c_int(N), c_int(K), c_int(_EPI[epilogue]), c_int(ks), ptr(ssq),
        c_int(0 if ssq is None else ssq.shape[1]), c_float(eps), ptr(None), ptr(None), ptr(None), stream()),
        "skinny_gemm_scaled")
    return out


def skinny_gemm_residual(x: torch.Tensor, w: torch.Tensor, h: torch.Tensor, gain: torch.Tensor, *,
                         ks: Optional[int] = None):
    """``h += x @ w.T`` in place (``h`` float32 ``[M, N]``), and what the RMSNorm after that sum needs: returns
    ``(bf16(h * gain) [M, N], ssq float32 [M, ceil(N / 16)])`` with ``ssq`` the sums of squares of the new ``h``
    over tiles of 16 columns.  ``skinny_gemm_scaled`` takes both."""
    require_cuda(x, w, h, gain)
    N, K = w.shape
    M = x.shape[0]
    if x.shape[1] != K or tuple(h.shape) != (M, N) or h.dtype != torch.float32 or not h.is_contiguous():
        raise KernelError("skinny_gemm_residual: h must be contiguous float32 [M, N]")
    if gain.dtype != torch.float32 or gain.numel() != N:
        raise KernelError("skinny_gemm_residual: gain must be float32 [N]")
    tiles = (N + 15) // 16
    out = torch.empty((M, N), dtype=torch.bfloat16, device=w.device)
    ssq = torch.empty((M, tiles), dtype=torch.float32, device=w.device)
    if ks is None:
        ks = pick_ks(tiles, K)
    check(fn("decode", "sx_skinny_gemm_norm")(
        ptr(x), ptr(w), ptr(out), c_int(M), c_int(N), c_int(K), c_int(3), c_int(ks), ptr(None), c_int(0),
        c_float(0.0), ptr(h), ptr(gain), ptr(ssq), stream()), "skinny_gemm_residual")
    return out, ssq


_SM_COUNT = {}


def sm_count(device) -> int:
    i = torch.device(device).index or 0
    if i not in _SM_COUNT:
        _SM_COUNT[i] = torch.cuda.get_device_properties(i).multi_processor_count
    return _SM_COUNT[i]
