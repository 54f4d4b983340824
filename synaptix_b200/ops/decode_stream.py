"""Python face of ``csrc/decode_stream.cu``: a run of decoder layers of a single-token step as one
persistent kernel (bfloat16, at most 8 sequences).

A ``StreamPlan`` is built once from the descriptions of consecutive layer runs (what their parts
report through ``stream_fields()``) and the cache they work on; ``run`` then advances the float32
residual stream through all of them with one launch.  ``StreamPlan.build`` returns ``None`` when
the kernel does not take the sizes; the caller then runs the layers kernel by kernel.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import List, Optional, Sequence

import torch

from ._lib import KernelError, c_int, c_ulonglong, check, fn, ptr, stream

MAX_ROWS = 8
_GROUPS = 4


class _Layer(ctypes.Structure):
    _fields_ = [("w_qkv", ctypes.c_void_p), ("w_o", ctypes.c_void_p), ("w_gu", ctypes.c_void_p),
                ("w_down", ctypes.c_void_p), ("g_in", ctypes.c_void_p), ("g_post", ctypes.c_void_p),
                ("g_q", ctypes.c_void_p), ("g_k", ctypes.c_void_p), ("inv_freq", ctypes.c_void_p),
                ("k_pages", ctypes.c_void_p), ("v_pages", ctypes.c_void_p),
                ("eps_in", ctypes.c_float), ("eps_post", ctypes.c_float), ("eps_qk", ctypes.c_float),
                ("scale_log2", ctypes.c_float),
                ("window", ctypes.c_int), ("group", ctypes.c_int), ("write_cache", ctypes.c_int),
                ("n_pages", ctypes.c_int)]


def enabled() -> bool:
    """``SYNAPTIX_STREAM=1`` in the environment turns the fused layer kernel on.  It is off by default:
    on a B200 a layer of the 4B shape takes 79 us in it at batch 1 against 61 us for the separate
    kernels (barriers across the grid and the single block per SM cost more than the kernel
    boundaries they replace)."""
    return os.environ.get("SYNAPTIX_STREAM", "0") == "1"


def grid_blocks(hd: int) -> int:
    """Blocks of the cooperative grid on the current device; 0 if the kernel cannot run there."""
    f = fn("decode_stream", "sx_decode_stream_blocks")
    return int(f(c_int(hd)))


def _addr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


class StreamPlan:
    """Consecutive layer runs with the same sizes, ready to launch."""

    def __init__(self, table: torch.Tensor, n_layers: int, H: int, nh: int, nkv: int, hd: int, I: int,
                 blocks: int, scratch: torch.Tensor, max_items: int, keep: list):
        self.table, self.n_layers = table, n_layers
        self.H, self.nh, self.nkv, self.hd, self.I = H, nh, nkv, hd, I
        self.blocks, self.scratch, self.max_items = blocks, scratch, max_items
        self._keep = keep            # the tensors whose addresses the table holds

    @staticmethod
    def build(layers: Sequence[dict], device) -> Optional["StreamPlan"]:
        """``layers``: one dict per run with the keys of ``_Layer`` as tensors and numbers, plus the
        sizes ``H, nh, nkv, hd, I``.  ``None`` if the sizes differ between runs or the kernel refuses them."""
        if not layers:
            return None
        H, nh, nkv, hd, I = (layers[0][k] for k in ("H", "nh", "nkv", "hd", "I"))
        if any((d["H"], d["nh"], d["nkv"], d["hd"], d["I"]) != (H, nh, nkv, hd, I) for d in layers):
            return None
        if hd not in (64, 128) or nh % nkv or nh // nkv > 16 or H % 32 or I % 32 or (nh * hd) % 32:
            return None
        if MAX_ROWS * (((H * 2 + 127) // 128) * 128 + 64) + 128 + 4096 > 104448:
            return None
        if any(d["group"] >= _GROUPS for d in layers):
            return None
        blocks = grid_blocks(hd)
        if blocks <= 0:
            return None
        arr = (_Layer * len(layers))()
        keep = []
        for i, d in enumerate(layers):
            e = arr[i]
            for name in ("w_qkv", "w_o", "w_gu", "w_down", "g_in", "g_post", "g_q", "g_k", "inv_freq", "k_pages", "v_pages"):
                t = d.get(name)
                if t is not None:
                    if not (t.is_cuda and t.is_contiguous()):
                        return None
                    keep.append(t)
                setattr(e, name, _addr(t))
            for name in ("w_qkv", "w_o", "w_gu", "w_down", "k_pages", "v_pages"):
                if d[name].dtype != torch.bfloat16:
                    return None
            e.eps_in, e.eps_post, e.eps_qk = d["eps_in"], d["eps_post"], d.get("eps_qk") or 0.0
            e.scale_log2 = d["scale"] * math.log2(math.e)
            e.window = int(d.get("window") or 0)
            e.group, e.write_cache = int(d["group"]), int(bool(d["write_cache"]))
            e.n_pages = int(d["k_pages"].shape[0])
        raw = bytes(arr)
        table = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device)
        max_items = max(blocks, MAX_ROWS * nkv)
        f = fn("decode_stream", "sx_decode_stream_scratch_bytes")
        f.restype = ctypes.c_ulonglong
        nbytes = int(f(c_int(nh), c_int(nkv), c_int(hd), c_int(I), c_int(max_items)))
        if nbytes <= 0:
            return None
        scratch = torch.zeros(nbytes + 256, dtype=torch.uint8, device=device)
        off = (-scratch.data_ptr()) % 256
        scratch = scratch[off:off + nbytes]
        return StreamPlan(table, len(layers), H, nh, nkv, hd, I, blocks, scratch, max_items, keep)

    def takes(self, rows: int) -> bool:
        return 0 < rows <= MAX_ROWS

    def run(self, h: torch.Tensor, positions: torch.Tensor, seq_lens: torch.Tensor,
            block_tables: Sequence[torch.Tensor], max_len: int, prof: Optional[torch.Tensor] = None) -> None:
        """Advances ``h`` (float32 ``[M, H]``, in place) through the plan's layer runs.  ``prof``: an
        int64 tensor ``[blocks, n_layers, 16]`` that receives the phases' time stamps (a tuning aid)."""
        M = h.shape[0]
        if h.dtype != torch.float32 or not h.is_contiguous() or h.shape[1] != self.H or not self.takes(M):
            raise KernelError("decode_stream: h must be contiguous float32 [M <= 8, H]")
        pages = max(1, (max_len + 63) // 64)
        n_splits = max(1, min(self.blocks // (M * self.nkv), pages, 512))
        bts = (ctypes.c_void_p * _GROUPS)()
        maxp = (ctypes.c_int * _GROUPS)()
        for g, bt in enumerate(block_tables):
            if g >= _GROUPS:
                break
            bts[g] = bt.data_ptr()
            maxp[g] = bt.shape[1]
        check(fn("decode_stream", "sx_decode_stream")(
            ptr(self.table), c_int(self.n_layers), c_int(M), c_int(self.H), c_int(self.nh), c_int(self.nkv),
            c_int(self.hd), c_int(self.I), ptr(h), ptr(positions), ptr(seq_lens), bts, maxp,
            ctypes.c_void_p(self.scratch.data_ptr()), c_ulonglong(self.scratch.numel()), c_int(self.max_items),
            c_int(n_splits), ptr(prof), stream()), "decode_stream")

    def status(self) -> int:
        """0, or 3 when a bounded wait at a grid barrier inside the kernel ran out.  Synchronises the device."""
        v = ctypes.c_int(0)
        check(fn("decode_stream", "sx_decode_stream_status")(
            ctypes.c_void_p(self.scratch.data_ptr()), c_int(self.nh), c_int(self.nkv), c_int(self.hd), c_int(self.I),
            c_int(self.max_items), ctypes.byref(v)), "decode_stream_status", launches=0)
        return int(v.value)
