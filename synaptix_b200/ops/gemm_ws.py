"""Python face of the weight-streaming tcgen05 product in ``csrc/gemm_ws.cu`` (bfloat16, up to 256 rows)."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from ._lib import KernelError, c_float, c_int, check, fn, ptr, require_cuda, stream

_EPI = {None: 0, "f32": 1, "silu_mul": 2, "residual": 3}
MAX_ROWS = 256


_RESIDUAL_PLANS = {}


def ws_supported(M: int, N: int, K: int, x_dtype, w_dtype) -> bool:
    return x_dtype == torch.bfloat16 and w_dtype == torch.bfloat16 and 0 < M <= MAX_ROWS and K > 0 and K % 8 == 0 and N > 0


def plan_ws(M: int, N: int, K: int, epilogue: Optional[str] = None) -> Tuple[int, int]:
    """``(tiles, splits)``: tiles of 128 columns of the result (64 with ``"silu_mul"``) and the blocks of a
    thread-block cluster that share a tile's K, as the library chooses them on the current device."""
    out = (ctypes.c_int * 2)()
    check(fn("gemm_ws", "sx_gemm_ws_plan")(c_int(M), c_int(N), c_int(K), c_int(_EPI[epilogue]), out), "gemm_ws_plan",
          launches=0)
    return int(out[0]), int(out[1])


def gemm_ws(x: torch.Tensor, w: torch.Tensor, *, epilogue: Optional[str] = None, ssq: Optional[torch.Tensor] = None,
            eps: float = 0.0, splits: Optional[int] = None, stages: Optional[int] = None,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x[M, K] @ w[N, K].T`` for ``M <= 256`` rows with ``w`` as the tensor cores' M side, read once from HBM;
    K is shared by the ``splits`` (1, 2, 4, 8) blocks of a cluster, which add up through their shared memory.

    ``epilogue``: ``None`` -> bfloat16 ``[M, N]``; ``"f32"`` -> float32; ``"silu_mul"`` -> ``w`` is ``[gate; up]``
    stacked, result bfloat16 ``[M, N/2]``.  With ``ssq`` (float32 ``[M, n]``) row ``m`` of the product is multiplied
    by ``rsqrt(sum(ssq[m]) / K + eps)`` before the epilogue: rows of ``x`` that lack their RMSNorm factor."""
    require_cuda(x, w, ssq, out)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError("gemm_ws: inner sizes differ")
    if epilogue not in (None, "f32", "silu_mul"):
        raise KernelError(f"gemm_ws: unknown epilogue {epilogue!r}")
    if not ws_supported(M, N, K, x.dtype, w.dtype):
        raise KernelError("gemm_ws: bfloat16 operands, at most 256 rows and K a multiple of 8")
    if ssq is not None and (ssq.dtype != torch.float32 or ssq.dim() != 2 or ssq.shape[0] != M):
        raise KernelError("gemm_ws: ssq must be float32 [M, n]")
    n_out = N // 2 if epilogue == "silu_mul" else N
    if out is None:
        out = torch.empty((M, n_out), dtype=torch.float32 if epilogue == "f32" else torch.bfloat16, device=x.device)
    check(fn("gemm_ws", "sx_gemm_ws")(ptr(x), ptr(w), ptr(out), c_int(M), c_int(N), c_int(K), c_int(_EPI[epilogue]),
                                      c_int(splits or 0), c_int(stages or 0), ptr(ssq), c_int(0 if ssq is None else ssq.shape[1]),
                                      c_float(eps), ptr(None), ptr(None), ptr(None), stream()), "gemm_ws")
    return out


def gemm_ws_residual(x: torch.Tensor, w: torch.Tensor, h: torch.Tensor, gain: torch.Tensor, *,
                     splits: Optional[int] = None, stages: Optional[int] = None):
    """``h += x @ w.T`` in place (``h`` float32 ``[M, N]``) and what the RMSNorm after that sum needs: returns
    ``(bf16(h * gain) [M, N], ssq float32 [M, n])`` with ``ssq`` sums of squares of the new ``h`` over each block's
    columns.  ``gemm_ws(..., ssq=ssq)`` takes both."""
    require_cuda(x, w, h, gain)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(h.shape) != (M, N) or h.dtype != torch.float32:
        raise KernelError("gemm_ws_residual: h must be contiguous float32 [M, N]")
    if gain.dtype != torch.float32 or gain.numel() != N:
        raise KernelError("gemm_ws_residual: gain must be float32 [N]")
    if not ws_supported(M, N, K, x.dtype, w.dtype):
        raise KernelError("gemm_ws_residual: bfloat16 operands, at most 256 rows and K a multiple of 8")
    plan = _RESIDUAL_PLANS.get((M, N, K))          # (a step asks dozens of times for two shapes)
    if plan is None:
        plan = _RESIDUAL_PLANS[(M, N, K)] = plan_ws(M, N, K, "residual")
    tiles, auto = plan
    splits = splits or auto
    while splits > (K + 63) // 64:
        splits //= 2
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    ssq = torch.empty((M, tiles * splits), dtype=torch.float32, device=x.device)
    check(fn("gemm_ws", "sx_gemm_ws")(ptr(x), ptr(w), ptr(out), c_int(M), c_int(N), c_int(K), c_int(3), c_int(splits),
                                      c_int(stages or 0), ptr(None), c_int(0), c_float(0.0), ptr(h), ptr(gain), ptr(ssq), stream()),
          "gemm_ws_residual")
    return out, ssq


def gemm_ws_status(reset: bool = False) -> int:
    """0, or which bounded wait of the kernel ran out (1 producer, 2 MMA issuer, 3 the warps that read the
    accumulator).  No device call: the word lies in host memory the device writes to."""
    v = ctypes.c_int(0)
    check(fn("gemm_ws", "sx_gemm_ws_status")(ctypes.byref(v), c_int(1 if reset else 0)), "gemm_ws_status", launches=0)
    return v.value
