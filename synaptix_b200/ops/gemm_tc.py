"""Python face of the tcgen05/TMEM/TMA matrix product in ``csrc/gemm_tc.cu`` (bfloat16)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ._lib import KernelError, c_int, check, fn, ptr, require_cuda, stream

_EPI = {None: 0, "f32": 1, "silu_mul": 2}


def tc_supported(M: int, N: int, K: int, x_dtype, w_dtype) -> bool:
    return x_dtype == torch.bfloat16 and w_dtype == torch.bfloat16 and K > 0 and K % 8 == 0 and M > 0 and N > 0


def gemm_tc(x: torch.Tensor, w: torch.Tensor, *, epilogue: Optional[str] = None,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x[M, K] @ w[N, K].T`` on the tcgen05 tensor cores, 32-bit accumulation in tensor memory.

    ``epilogue``: ``None`` -> bfloat16 ``[M, N]``; ``"f32"`` -> float32 ``[M, N]``; ``"silu_mul"`` ->
    ``w`` is ``[gate; up]`` stacked and the result is bfloat16 ``[M, N/2]``.  Needs ``K % 8 == 0``.
    """
    require_cuda(x, w, out)
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError("gemm_tc: inner sizes differ")
    if not tc_supported(M, N, K, x.dtype, w.dtype):
        raise KernelError("gemm_tc: bfloat16 operands and K a multiple of 8")
    if epilogue not in _EPI:
        raise KernelError(f"gemm_tc: unknown epilogue {epilogue!r}")
    n_out = N // 2 if epilogue == "silu_mul" else N
    if out is None:
        out = torch.empty((M, n_out), dtype=torch.float32 if epilogue == "f32" else torch.bfloat16, device=x.device)
    check(fn("gemm_tc", "sx_gemm_tc")(ptr(x), ptr(w), ptr(out), c_int(M), c_int(N), c_int(K), c_int(_EPI[epilogue]),
                                      stream()), "gemm_tc")
    return out


def gemm_tc_status() -> int:
    """0, or which bounded wait of the kernel ran out (1 producer, 2 MMA issuer, 3 epilogue); synchronises."""
    v = ctypes.c_int(0)
    check(fn("gemm_tc", "sx_gemm_tc_status")(ctypes.byref(v)), "gemm_tc_status", launches=0)
    return v.value
