"""Python face of the tcgen05/TMEM/TMA matrix product in ``csrc/gemm_tc.cu`` (bfloat16)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ._lib import KernelError, c_int, check, fn, ptr, require_cuda, stream
from .decode import sm_count

_EPI = {None: 0, "f32": 1, "silu_mul": 2}


def tc_supported(M: int, N: int, K: int, x_dtype, w_dtype) -> bool:
    return x_dtype == torch.bfloat16 and w_dtype == torch.bfloat16 and K > 0 and K % 8 == 0 and M > 0 and N > 0


def plan_splits(M: int, N: int, K: int, n_sm: int) -> int:
    """How many blocks split K: 1 when whole 128 x 256 tiles already fill the GPU, else enough
    128 x 128 tiles x splits to give every SM a block (each split at least two 64-wide slices)."""
    tiles_256 = ((N + 255) // 256) * ((M + 127) // 128)
    if tiles_256 >= (n_sm * 3) // 4:
        return 1
    tiles_128 = ((N + 127) // 128) * ((M + 127) // 128)
    nkb = (K + 63) // 64
    return max(1, min(nkb // 2, (n_sm + tiles_128 // 2) // tiles_128))


_TAIL_COUNTS = {}


def _tail_counts(device) -> torch.Tensor:
    """Zeroed int32 counters, one array per device; the kernel leaves them zero."""
    key = torch.device(device).index or 0
    if key not in _TAIL_COUNTS:
        _TAIL_COUNTS[key] = torch.zeros(1024, dtype=torch.int32, device=device)
    return _TAIL_COUNTS[key]


def plan_tail(M: int, N: int, K: int, n_sm: int):
    """``(tail_tiles, tail_splits)``: how many of the LAST 128 x 256 tiles are computed as several work items
    that split K, and into how many.  The persistent kernel runs one block per SM
    over whole tiles; when the tiles of the last round would keep at most a quarter of the SMs busy (2,048
    rows by 2,560 columns: 160 tiles on 148 SMs), that round costs a full tile's time for little work.
    The tail is the bottom of the last column of tiles, so it must fit there; ``(0, 0)`` otherwise."""
    tiles_m, tiles_n = (M + 127) // 128, (N + 255) // 256
    n_tiles = tiles_m * tiles_n
    rem = n_tiles % n_sm
    if n_tiles <= n_sm or rem == 0 or rem > n_sm // 4 or rem > tiles_m or rem > 512:
        return 0, 0
    nkb = (K + 63) // 64
    splits = max(1, min(nkb // 2, n_sm // rem))
    return (rem, splits) if splits >= 2 else (0, 0)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, *, epilogue: Optional[str] = None,
            out: Optional[torch.Tensor] = None, splits: Optional[int] = None,
            tail: Optional[bool] = None) -> torch.Tensor:
    """``x[M, K] @ w[N, K].T`` on the tcgen05 tensor cores, 32-bit accumulation in tensor memory.

    ``splits``: blocks that split K (default: chosen so that the GPU is filled; more than one only
    matters for few rows).  With ``splits > 1`` float32 partial tiles go through a workspace of
    ``splits * M * N`` floats and a second kernel adds them in a fixed order.

    ``tail`` (default: on, ``False`` turns it off): see ``plan_tail``.

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
    if splits is None:
        splits = plan_splits(M, N, K, sm_count(x.device))
    splits = max(1, min(int(splits), (K + 63) // 64))
    tail_tiles = tail_splits = 0
    if splits == 1 and epilogue != "silu_mul" and tail is not False:
        tail_tiles, tail_splits = plan_tail(M, N, K, sm_count(x.device))
    ws = None
    if splits > 1:
        ws = torch.empty(splits * M * N, dtype=torch.float32, device=x.device)
    elif tail_tiles:
        m_rows, n_cols = M - ((M + 127) // 128 - tail_tiles) * 128, N - ((N + 255) // 256 - 1) * 256
        ws = torch.empty(tail_splits * m_rows * n_cols, dtype=torch.float32, device=x.device)
    check(fn("gemm_tc", "sx_gemm_tc")(ptr(x), ptr(w), ptr(out), c_int(M), c_int(N), c_int(K), c_int(_EPI[epilogue]),
                                      c_int(splits), ptr(ws), c_int(tail_tiles), c_int(tail_splits),
                                      ptr(_tail_counts(x.device) if tail_tiles else None), stream()), "gemm_tc",
          launches=2 if splits > 1 else 1)
    return out


def gemm_tc_status() -> int:
    """0, or which bounded wait of the kernel ran out (1 producer, 2 MMA issuer, 3 epilogue); synchronises."""
    v = ctypes.c_int(0)
    check(fn("gemm_tc", "sx_gemm_tc_status")(ctypes.byref(v)), "gemm_tc_status", launches=0)
    return v.value
