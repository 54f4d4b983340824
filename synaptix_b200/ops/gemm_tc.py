"""Python face of the tcgen05/TMEM/TMA matrix product in ``csrc/gemm_tc.cu`` (bfloat16)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ._lib import KernelError, c_int, check, fn, ptr, require_cuda, stream
from .decode import sm_count
from .options import OPTIONS

_EPI = {None: 0, "f32": 1, "silu_mul": 2}


def tc_supported(M: int, N: int, K: int, x_dtype, w_dtype) -> bool:
    return x_dtype == torch.bfloat16 and w_dtype == torch.bfloat16 and K > 0 and K % 8 == 0 and M > 0 and N > 0


_COUNTS = {}


def _counts(device) -> torch.Tensor:
    """Zeroed int32 counters, one array per device; the kernel leaves them zero."""
    key = torch.device(device).index or 0
    if key not in _COUNTS:
        _COUNTS[key] = torch.zeros(2048, dtype=torch.int32, device=device)
    return _COUNTS[key]


def plan_splits(M: int, N: int, K: int, n_sm: int) -> int:
    """Blocks that split K in the two-kernel form, for products with only a handful of 128 x 256 tiles (few rows
    and a narrow matrix): 1 when whole tiles already fill three quarters of the GPU, else enough 128 x 128
    tiles x splits to give every SM a block (each split at least two 64-wide slices)."""
    tiles_256 = ((N + 255) // 256) * ((M + 127) // 128)
    if tiles_256 >= (n_sm * 3) // 4:
        return 1
    # several rows of tiles: beyond a dozen tiles whole ones measured faster than this form wherever the persistent
    # kernel does not cut them itself (256 x 6,144 x 2,560: 20.5 against 35.1 us; 512 x 2,560 x 4,096: 27.7 against 40.3)
    if M > 128 and tiles_256 > 12:
        return 1
    tiles_128 = ((N + 127) // 128) * ((M + 127) // 128)
    nkb = (K + 63) // 64
    return max(1, min(nkb // 2, (n_sm + tiles_128 // 2) // tiles_128))


_PLANS = {}
_WORKSPACES = {}


def _workspace(n_floats: int, device) -> torch.Tensor:
    """Float32 scratch for partial tiles.  One buffer per device that only grows: the kernels of a stream run one
    after the other, and a partial tile is read by the launch (or the second kernel) that wrote it.  While a CUDA
    graph is being captured a fresh buffer is taken instead (it belongs to that graph's memory)."""
    if torch.cuda.is_current_stream_capturing():
        return torch.empty(n_floats, dtype=torch.float32, device=device)
    key = torch.device(device).index or 0
    buf = _WORKSPACES.get(key)
    if buf is None or buf.numel() < n_floats:
        buf = _WORKSPACES[key] = torch.empty(max(n_floats, 1 << 22), dtype=torch.float32, device=device)
    return buf


_cut_few_applied = None


def _apply_cut_few() -> None:
    """Hand option ``gemm_cut_few`` to the library when it changed."""
    global _cut_few_applied
    if _cut_few_applied != OPTIONS.gemm_cut_few:
        fn("gemm_tc", "sx_gemm_tc_cut_few")(c_int(1 if OPTIONS.gemm_cut_few else 0))
        _cut_few_applied = OPTIONS.gemm_cut_few


def plan_stream(M: int, N: int, K: int, epilogue: Optional[str] = None):
    """``(whole tiles, cut tiles, most pieces a cut tile has, grid)`` of the persistent kernel on the current
    device.  Tiles that would not fill a round of all SMs (a last round at most half full: 2,048 x 2,560 has
    160 tiles for 148 SMs; or all tiles of a step with at most 128 rows) are cut over K: their 64-wide slices
    of K form one sequence that is dealt out to the blocks in equal contiguous shares, the blocks of a tile
    leave float32 partial tiles in a workspace and add them up together, in a fixed order.  Several rows of tiles
    that are fewer than the SMs (a few hundred rows) are cut when an estimate from measured times says that pays
    (option ``gemm_cut_few``)."""
    _apply_cut_few()
    out = (ctypes.c_int * 4)()
    check(fn("gemm_tc", "sx_gemm_tc_plan")(c_int(M), c_int(N), c_int(K), c_int(_EPI[epilogue]), out), "gemm_tc_plan",
          launches=0)
    return tuple(int(v) for v in out)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, *, epilogue: Optional[str] = None,
            out: Optional[torch.Tensor] = None, splits: Optional[int] = None,
            cut: Optional[bool] = None) -> torch.Tensor:
    """``x[M, K] @ w[N, K].T`` on the tcgen05 tensor cores, 32-bit accumulation in tensor memory.

    Default: the persistent kernel, which cuts tiles over K where whole tiles would leave SMs idle (see
    ``plan_stream``; ``cut=False`` turns that off); for a handful of tiles the two-kernel form instead
    (``plan_splits``).  ``splits > 1`` asks for that form: K split over ``splits`` blocks per 128 x 128 tile,
    float32 partial tiles in a workspace of ``splits * M * N`` floats, added in a fixed order by a second kernel;
    ``splits=1`` for whole tiles (or cut ones) in any case.

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
    ws = counts = None
    if cut is None:
        cut = OPTIONS.gemm_cut
    _apply_cut_few()
    # what the library will do with this shape, remembered: a prompt step asks a hundred times for a handful of shapes
    key = (M, N, K, epilogue, splits, bool(cut), OPTIONS.gemm_cut_few)
    plan = _PLANS.get(key)
    if plan is None:
        n_cut = zmax = 0
        if splits is None and cut is not False:
            _, n_cut, zmax, _ = plan_stream(M, N, K, epilogue)
        sp = splits
        if sp is None:
            sp = 1 if n_cut else plan_splits(M, N, K, sm_count(x.device))
        sp = max(1, min(int(sp), (K + 63) // 64))
        plan = _PLANS[key] = (sp, n_cut, sp * M * N if sp > 1 else n_cut * zmax * 128 * 256)
    splits, n_cut, ws_floats = plan
    if ws_floats:
        ws = _workspace(ws_floats, x.device)
        if splits == 1:
            counts = _counts(x.device)
    check(fn("gemm_tc", "sx_gemm_tc")(ptr(x), ptr(w), ptr(out), c_int(M), c_int(N), c_int(K), c_int(_EPI[epilogue]),
                                      c_int(splits), ptr(ws), ctypes.c_ulonglong(0 if ws is None else ws.numel()),
                                      ptr(counts), stream()), "gemm_tc", launches=2 if splits > 1 else 1)
    return out


QKV_HEAD_DIM = 128


def qkv_epilogue_supported(M: int, nh: int, nkv: int, hd: int, K: int, x_dtype, w_dtype) -> bool:
    """Can the fused q/k/v projection prepare the heads in its epilogue?  Heads of 128, an even number of them
    (a 256-wide tile holds two), bfloat16."""
    return (x_dtype == torch.bfloat16 and w_dtype == torch.bfloat16 and hd == QKV_HEAD_DIM and (nh + 2 * nkv) % 2 == 0
            and K > 0 and K % 8 == 0 and M > 0)


def gemm_tc_qkv(x: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, k_pages: Optional[torch.Tensor],
                v_pages: Optional[torch.Tensor], wq: Optional[torch.Tensor], wk: Optional[torch.Tensor],
                cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], eps: float, positions: torch.Tensor,
                seq_of_token: torch.Tensor, block_table: torch.Tensor, nh: int, nkv: int) -> None:
    """``x @ w.T`` for the stacked q/k/v matrix with heads of 128, and what ``qkv_prepare`` does to the result, in
    the product's epilogue: per-head RMSNorm of q and k (gains ``wq`` / ``wk``, skipped when ``None``), rotate-half
    rotation by the angles whose cosines and sines are ``cos`` / ``sin [M, 64]`` (skipped when ``None``), q to
    ``q_out [M, nh * 128]``, k and v into the pages (skipped when ``None``)."""
    require_cuda(x, w, q_out, k_pages, v_pages, wq, wk, cos, sin, positions, seq_of_token, block_table)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or N != (nh + 2 * nkv) * QKV_HEAD_DIM or not qkv_epilogue_supported(M, nh, nkv, QKV_HEAD_DIM, K, x.dtype, w.dtype):
        raise KernelError("gemm_tc_qkv: bfloat16, heads of 128, an even number of heads, K a multiple of 8")
    if q_out.dtype != torch.bfloat16 or tuple(q_out.shape) != (M, nh * QKV_HEAD_DIM):
        raise KernelError("gemm_tc_qkv: q_out must be bfloat16 [M, nh * 128]")
    n_pages = 0
    for pg in (k_pages, v_pages):
        if pg is not None:
            if pg.dtype != torch.bfloat16 or pg.dim() != 4 or tuple(pg.shape[1:]) != (nkv, 64, QKV_HEAD_DIM):
                raise KernelError("gemm_tc_qkv: cache pages must be bfloat16 [n_pages, nkv, 64, 128]")
            n_pages = pg.shape[0]
    for t in (wq, wk):
        if t is not None and (t.dtype != torch.float32 or t.numel() != QKV_HEAD_DIM):
            raise KernelError("gemm_tc_qkv: norm gains are float32 [128]")
    if (cos is None) != (sin is None) or (cos is not None and (cos.dtype != torch.float32 or tuple(cos.shape) != (M, 64)
                                                                 or tuple(sin.shape) != (M, 64))):
        raise KernelError("gemm_tc_qkv: cos and sin are float32 [M, 64]")
    for t in (positions, seq_of_token, block_table):
        if t.dtype != torch.int32:
            raise KernelError("gemm_tc_qkv: index tensors are int32")
    check(fn("gemm_tc", "sx_gemm_tc_qkv")(
        ptr(x), ptr(w), c_int(M), c_int(N), c_int(K), ptr(q_out), ptr(k_pages), ptr(v_pages), ptr(wq), ptr(wk), ptr(cos),
        ptr(sin), ptr(positions), ptr(seq_of_token), ptr(block_table), c_int(block_table.shape[1]), c_int(nh), c_int(nkv),
        c_int(n_pages), ctypes.c_float(eps), stream()), "gemm_tc_qkv")


def gemm_tc_status(reset: bool = False) -> int:
    """0, or which bounded wait of the kernel ran out (1 producer, 2 and 4 MMA issuer, 3 epilogue, 5 the blocks
    of a cut tile waiting for one another).  The word lies in host memory the device writes to, so this is no
    device call; it tells of launches the host has already waited for.  ``reset`` puts it back to 0 and zeroes
    the counters of cut tiles, which a wait that ran out may have left non-zero."""
    v = ctypes.c_int(0)
    check(fn("gemm_tc", "sx_gemm_tc_status")(ctypes.byref(v), c_int(1 if reset else 0)), "gemm_tc_status", launches=0)
    if reset and v.value:
        for t in _COUNTS.values():
            t.zero_()
    return v.value
