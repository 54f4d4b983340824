"""Python faces of the tensor-core attention kernels in ``csrc/attention.cu`` (bfloat16)."""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

import ctypes

from ._lib import KernelError, c_float, c_int, c_longlong, check, fn, ptr, require_cuda, stream
from .decode import sm_count
from .options import OPTIONS

FAST_HEAD_DIMS = (32, 64, 128)


def fast_supported(dtype, nh: int, nkv: int, hd: int) -> bool:
    return dtype == torch.bfloat16 and hd in FAST_HEAD_DIMS and nkv > 0 and nh % nkv == 0 and nh // nkv <= 16


def pick_splits(n_seqs: int, nkv: int, max_pages: int, device) -> int:
    """Splits of a sequence's pages over blocks: as many as keep all blocks in ONE wave (two
    blocks fit an SM), since a second, partly filled wave costs as much as a full one; then
    no more than give every split a page (a kernel cuts ``ceil(pages / splits)`` pages a split:
    37 splits of 64 pages are 32 splits of 2 pages and 5 empty blocks, measured 12.5 against 10.3 us)."""
    slots = 2 * sm_count(device)
    base = max(1, n_seqs * nkv)
    s = max(1, min(max_pages, slots // base))
    per = -(-max_pages // s)
    return max(1, -(-max_pages // per))


_COUNTERS = {}
_MAX_COUNTERS = 1 << 16


def _counters(device) -> torch.Tensor:
    """Zeroed int32 counters of finished blocks, one array per device; every launch leaves them zero."""
    key = torch.device(device).index or 0
    if key not in _COUNTERS:
        _COUNTERS[key] = torch.zeros(_MAX_COUNTERS, dtype=torch.int32, device=device)
    return _COUNTERS[key]


def attn_decode(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, seq_lens: torch.Tensor,
                block_table: torch.Tensor, nh: int, nkv: int, hd: int, scale: float, window: Optional[int],
                n_splits: int, out: Optional[torch.Tensor] = None,
                scratch: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, fused_merge: bool = False) -> torch.Tensor:
    """One query token per sequence (row ``s`` of ``q`` belongs to sequence ``s``) against the
    sequence's ``seq_lens[s]`` cached keys (its own included).  ``n_splits > 1`` splits the
    pages of every sequence over blocks; partial results go through float32 scratch
    (``scratch = (part_o [S*nh*n_splits*hd], part_ml [S*nh*n_splits*2])``, allocated if absent).
    With ``fused_merge`` the block of a (sequence, kv head) that finishes last merges the splits
    inside the kernel; otherwise (the default: it measured faster, 3.96 against 4.08 ms for a
    batch-8 step of the 4B shape) a second kernel does."""
    require_cuda(q, k_pages, v_pages, seq_lens, block_table, out)
    S = q.shape[0]
    if not fast_supported(q.dtype, nh, nkv, hd) or k_pages.dtype != q.dtype:
        raise KernelError("attn_decode: bfloat16, head size 32/64/128 and at most 16 query heads per kv head")
    if out is None:
        out = torch.empty((S, nh * hd), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if n_splits > 1:
        if scratch is None:
            part_o = torch.empty(S * nh * n_splits * hd, dtype=torch.float32, device=q.device)
            part_ml = torch.empty(S * nh * n_splits * 2, dtype=torch.float32, device=q.device)
        else:
            part_o, part_ml = scratch
            if part_o.numel() < S * nh * n_splits * hd or part_ml.numel() < S * nh * n_splits * 2:
                raise KernelError("attn_decode: scratch is too small")
    if fused_merge and n_splits > 1 and S * nkv <= _MAX_COUNTERS and n_splits <= 512:
        check(fn("attention", "sx_attn_decode_fused")(
            ptr(q), ptr(k_pages), ptr(v_pages), ptr(out), ptr(part_o), ptr(part_ml), ptr(_counters(q.device)),
            ptr(seq_lens), ptr(block_table), c_int(block_table.shape[1]), c_int(S), c_int(nh), c_int(nkv), c_int(hd),
            c_float(scale), c_int(0 if window is None else int(window)), c_int(n_splits), stream()), "attn_decode")
        return out
    check(fn("attention", "sx_attn_decode")(
        ptr(q), ptr(k_pages), ptr(v_pages), ptr(out), ptr(part_o), ptr(part_ml), ptr(seq_lens), ptr(block_table),
        c_int(block_table.shape[1]), c_int(S), c_int(nh), c_int(nkv), c_int(hd), c_float(scale),
        c_int(0 if window is None else int(window)), c_int(n_splits), stream()), "attn_decode",
        launches=2 if n_splits > 1 else 1)
    return out


def attn_decode_prep(qkv: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, seq_lens: torch.Tensor,
                     block_table: torch.Tensor, nh: int, nkv: int, hd: int, scale: float, window: Optional[int],
                     n_splits: int, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor],
                     inv_freq: Optional[torch.Tensor], eps: float, write_cache: bool,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``attn_decode`` straight from the step's fused projection ``qkv [S, (nh + 2 nkv) hd]``: the kernel
    normalises and rotates the query heads and the new key itself (what ``qkv_prepare`` does), writes the new key
    and value into the cache (``write_cache``) and attends.  The rotation is of the whole head or none."""
    require_cuda(qkv, k_pages, v_pages, seq_lens, block_table, out, wq, wk, inv_freq)
    S = qkv.shape[0]
    if not fast_supported(qkv.dtype, nh, nkv, hd) or k_pages.dtype != qkv.dtype or qkv.shape[1] != (nh + 2 * nkv) * hd:
        raise KernelError("attn_decode_prep: bfloat16 [S, (nh + 2 nkv) hd], head size 32/64/128, at most 16 query heads per kv head")
    if inv_freq is not None and inv_freq.numel() != hd // 2:
        raise KernelError("attn_decode_prep: the rotation must cover the whole head")
    if out is None:
        out = torch.empty((S, nh * hd), dtype=qkv.dtype, device=qkv.device)
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.empty(S * nh * n_splits * hd, dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty(S * nh * n_splits * 2, dtype=torch.float32, device=qkv.device)
    check(fn("attention", "sx_attn_decode_prep")(
        ptr(qkv), ptr(k_pages), ptr(v_pages), ptr(out), ptr(part_o), ptr(part_ml), ptr(wq), ptr(wk), ptr(inv_freq),
        c_float(eps), c_int(1 if write_cache else 0), c_longlong(k_pages.shape[0]), ptr(seq_lens), ptr(block_table),
        c_int(block_table.shape[1]), c_int(S), c_int(nh), c_int(nkv), c_int(hd), c_float(scale),
        c_int(0 if window is None else int(window)), c_int(n_splits), stream()), "attn_decode_prep",
        launches=2 if n_splits > 1 else 1)
    return out


TMA_HEAD_DIMS = (64, 128)
CLUSTER_SPLITS = (2, 4, 8, 16)          # split counts whose blocks can merge among themselves as a thread-block cluster
CLUSTER_SPLITS_USED = (2, 4)            # ... and those for which that measured faster than scratch and a second kernel


def use_cluster(n_splits: int) -> bool:
    """Should the splits of a (sequence, kv head) merge among themselves as a thread-block cluster?  Measured at
    32 query heads over 8 kv heads of 128, context 4,096, us a layer: 8 sequences, 4 splits 27.3 against 29.0 with
    the second kernel; but 1 sequence, 8 or 16 blocks a cluster 11.3 / 11.9 against 8.9 for 32 splits and a
    second kernel (a large cluster waits for as many free SMs of one GPC at once, and fewer splits mean more
    pages one after another in a block): only small clusters are used."""
    return n_splits in CLUSTER_SPLITS_USED


def tma_decode_supported(dtype, nh: int, nkv: int, hd: int) -> bool:
    """The TMA-fed decode attention takes bfloat16, head size 64 or 128, at most 16 query heads per kv head."""
    return fast_supported(dtype, nh, nkv, hd) and hd in TMA_HEAD_DIMS


def attn_decode_tma(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, seq_lens: torch.Tensor,
                    block_table: torch.Tensor, nh: int, nkv: int, hd: int, scale: float, window: Optional[int],
                    n_splits: int, *, prep: bool = False, wq: Optional[torch.Tensor] = None,
                    wk: Optional[torch.Tensor] = None, inv_freq: Optional[torch.Tensor] = None, eps: float = 0.0,
                    write_cache: bool = True, out: Optional[torch.Tensor] = None,
                    cluster: Optional[bool] = None) -> torch.Tensor:
    """Single-token attention with pages brought by TMA and a warp per page (``csrc/attn_decode.cu``).

    ``q`` is ``[S, nh * hd]`` prepared queries against a cache that already holds the step's keys and values;
    or, with ``prep``, the step's fused projection ``[S, (nh + 2 nkv) hd]``: the kernel then normalises (gains
    ``wq``/``wk``, ``eps``) and rotates (``inv_freq``: the whole head, or ``None``) the query heads and the new
    key itself and, with ``write_cache``, stores the new key and value.  ``n_splits`` blocks share a
    sequence's pages; with 2, 4, 8 or 16 of them and ``cluster`` they merge their partial results among
    themselves as a thread-block cluster, otherwise through scratch memory and a second kernel.  ``cluster=None``
    decides by ``use_cluster``."""
    require_cuda(q, k_pages, v_pages, seq_lens, block_table, out, wq, wk, inv_freq)
    S = q.shape[0]
    if not tma_decode_supported(q.dtype, nh, nkv, hd) or k_pages.dtype != q.dtype:
        raise KernelError("attn_decode_tma: bfloat16, head size 64 or 128 and at most 16 query heads per kv head")
    if q.shape[1] != ((nh + 2 * nkv) * hd if prep else nh * hd):
        raise KernelError("attn_decode_tma: q has the wrong width")
    if inv_freq is not None and inv_freq.numel() != hd // 2:
        raise KernelError("attn_decode_tma: the rotation must cover the whole head")
    if out is None:
        out = torch.empty((S, nh * hd), dtype=q.dtype, device=q.device)
    n_splits = max(1, int(n_splits))
    part_o = part_ml = None
    clustered = (use_cluster(n_splits) if cluster is None else bool(cluster)) and n_splits in CLUSTER_SPLITS
    if n_splits > 1 and not clustered:
        part_o = torch.empty(S * nh * n_splits * hd, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(S * nh * n_splits * 2, dtype=torch.float32, device=q.device)
    check(fn("attn_decode", "sx_attn_decode_tma")(
        ptr(q), ptr(k_pages), ptr(v_pages), ptr(out), ptr(part_o), ptr(part_ml), c_int(1 if prep else 0), ptr(wq),
        ptr(wk), ptr(inv_freq), c_float(eps), c_int(1 if write_cache else 0), c_longlong(k_pages.shape[0]),
        ptr(seq_lens), ptr(block_table), c_int(block_table.shape[1]), c_int(S), c_int(nh), c_int(nkv), c_int(hd),
        c_float(scale), c_int(0 if window is None else int(window)), c_int(n_splits), stream()), "attn_decode_tma",
        launches=2 if n_splits > 1 and not clustered else 1)
    return out


def attn_decode_status(reset: bool = False) -> int:
    """0, or which bounded wait of the TMA-fed decode attention ran out (1 the producer's, 2 a compute warp's).
    No device call; it tells of launches the host has already waited for.  ``reset`` puts it back to 0."""
    v = ctypes.c_int(0)
    check(fn("attn_decode", "sx_attn_decode_status")(ctypes.byref(v), c_int(1 if reset else 0)), "attn_decode_status",
          launches=0)
    return int(v.value)


def query_tiles(cu_seqlens: Sequence[int], rows: int = 64):
    """Lists (sequence, first row) of the ``rows``-row query tiles of a packed batch."""
    seqs, q0s = [], []
    for s in range(len(cu_seqlens) - 1):
        n = cu_seqlens[s + 1] - cu_seqlens[s]
        for q0 in range(0, n, rows):
            seqs.append(s)
            q0s.append(q0)
    return seqs, q0s


def attn_prefill(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, tile_seq: torch.Tensor,
                 tile_q0: torch.Tensor, cu_seqlens: torch.Tensor, seq_past: torch.Tensor, seq_lens: torch.Tensor,
                 block_table: torch.Tensor, nh: int, nkv: int, hd: int, scale: float, window: Optional[int],
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Packed query tokens of sequences with unequal lengths against the cache (which already
    holds this step's keys); ``tile_seq``/``tile_q0`` list the 64-row query tiles."""
    require_cuda(q, k_pages, v_pages, tile_seq, tile_q0, cu_seqlens, seq_past, seq_lens, block_table, out)
    T = q.shape[0]
    if not (q.dtype == torch.bfloat16 and hd in FAST_HEAD_DIMS and nh % nkv == 0):
        raise KernelError("attn_prefill: bfloat16 and head size 32/64/128")
    if out is None:
        out = torch.empty((T, nh * hd), dtype=q.dtype, device=q.device)
    check(fn("attention", "sx_attn_prefill")(
        ptr(q), ptr(k_pages), ptr(v_pages), ptr(out), ptr(tile_seq), ptr(tile_q0), c_int(tile_seq.numel()),
        ptr(cu_seqlens), ptr(seq_past), ptr(seq_lens), ptr(block_table), c_int(block_table.shape[1]), c_int(nh),
        c_int(nkv), c_int(hd), c_float(scale), c_int(0 if window is None else int(window)), stream()), "attn_prefill")
    return out


TC_HEAD_DIM = 128
TC_TILE_ROWS = 128


def tc_prefill_supported(dtype, nh: int, nkv: int, hd: int) -> bool:
    """The tcgen05 prompt-attention kernel takes bfloat16 and head size 128 (option ``attn_tc``)."""
    return dtype == torch.bfloat16 and hd == TC_HEAD_DIM and nkv > 0 and nh % nkv == 0 and OPTIONS.attn_tc


def attn_prefill_tc(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, tile_seq: torch.Tensor,
                    tile_q0: torch.Tensor, cu_seqlens: torch.Tensor, seq_past: torch.Tensor, seq_lens: torch.Tensor,
                    block_table: torch.Tensor, nh: int, nkv: int, hd: int, scale: float, window: Optional[int],
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``attn_prefill`` on the tcgen05 tensor cores (``csrc/attn_tc.cu``); ``tile_seq``/``tile_q0`` list
    128-row query tiles."""
    require_cuda(q, k_pages, v_pages, tile_seq, tile_q0, cu_seqlens, seq_past, seq_lens, block_table, out)
    T = q.shape[0]
    if not tc_prefill_supported(q.dtype, nh, nkv, hd) or k_pages.dtype != q.dtype:
        raise KernelError("attn_prefill_tc: bfloat16 and head size 128")
    if out is None:
        out = torch.empty((T, nh * hd), dtype=q.dtype, device=q.device)
    check(fn("attn_tc", "sx_attn_prefill_tc")(
        ptr(q), ptr(k_pages), ptr(v_pages), ptr(out), c_longlong(T), c_longlong(k_pages.shape[0]), ptr(tile_seq),
        ptr(tile_q0), c_int(tile_seq.numel()), ptr(cu_seqlens), ptr(seq_past), ptr(seq_lens), ptr(block_table),
        c_int(block_table.shape[1]), c_int(nh), c_int(nkv), c_int(hd), c_float(scale),
        c_int(0 if window is None else int(window)), stream()), "attn_prefill_tc")
    return out


def attn_tc_status(reset: bool = False) -> int:
    """0, or which bounded wait of the tcgen05 attention kernel ran out (1 producer, 2-5 MMA issuer, 6-9
    softmax).  No device call (the word lies in host memory the device writes to); it tells of launches the host
    has already waited for.  ``reset`` puts it back to 0."""
    v = ctypes.c_int(0)
    check(fn("attn_tc", "sx_attn_tc_status")(ctypes.byref(v), c_int(1 if reset else 0)), "attn_tc_status", launches=0)
    return int(v.value)
