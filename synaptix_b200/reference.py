"""The kernels' plain C++ counterparts on the CPU (``csrc/reference.cpp``), called with CPU tensors.

One function per kernel entry point, with the same arguments and the same meaning, written as naive
loops: they say what each kernel computes, and the tests compare every CUDA kernel with them (and them
with the plain Python implementation under ``tests/``).  Nothing in the package calls this module: the
product path has no CPU code.  The reference keeps such counterparts in a crate of their own
(crates/synaptix-kernels-cpu/src/lib.rs).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc.build import load_host_library

_DT = {torch.float32: 0, torch.bfloat16: 1}
_ERRORS = {10001: "unsupported dtype", 10002: "unsupported size"}


class ReferenceError_(RuntimeError):
    pass


def _fn(name: str):
    f = getattr(load_host_library("reference"), name)
    f.restype = ctypes.c_int
    return f


def _p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    if t.is_cuda or not t.is_contiguous():
        raise ReferenceError_("the C++ reference takes contiguous CPU tensors")
    return ctypes.c_void_p(t.data_ptr())


def _check(code: int, what: str) -> None:
    if code:
        raise ReferenceError_(f"{what}: {_ERRORS.get(code, code)}")


def _i32(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.int32).contiguous()


c_int, c_float = ctypes.c_int, ctypes.c_float


def embed_gather(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    V, H = table.shape
    ids = _i32(ids)
    out = torch.empty((ids.numel(), H), dtype=torch.float32)
    _check(_fn("sx_ref_embed_gather")(_p(table), c_int(_DT[table.dtype]), _p(ids), _p(out), c_int(ids.numel()), c_int(H),
                                      c_int(V)), "embed_gather")
    return out


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor, eps: float, dtype: torch.dtype,
                rows: Optional[torch.Tensor] = None, write_h: bool = True) -> torch.Tensor:
    """``h`` (float32, changed in place when ``delta`` is given and ``write_h``) -> normalised rows in ``dtype``."""
    T, H = h.shape
    if rows is not None:
        rows = _i32(rows)
    R = T if rows is None else rows.numel()
    y = torch.empty((R, H), dtype=dtype)
    _check(_fn("sx_ref_add_rmsnorm")(_p(h), _p(delta), _p(gain), c_float(eps), _p(y), _p(rows), c_int(R), c_int(H),
                                     c_int(_DT[dtype]), c_int(1 if write_h else 0)), "add_rmsnorm")
    return y


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> None:
    _check(_fn("sx_ref_residual_add")(_p(h), _p(delta), ctypes.c_longlong(h.numel()), c_int(_DT[delta.dtype])), "residual_add")


def gemm(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x[M, K] @ w[N, K].T``."""
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=out_dtype or x.dtype)
    _check(_fn("sx_ref_gemm")(_p(x), c_int(_DT[x.dtype]), _p(w), c_int(_DT[w.dtype]), _p(out), c_int(_DT[out.dtype]), c_int(M),
                              c_int(N), c_int(K)), "gemm")
    return out


def silu_mul(gu: torch.Tensor) -> torch.Tensor:
    T, I2 = gu.shape
    out = torch.empty((T, I2 // 2), dtype=gu.dtype)
    _check(_fn("sx_ref_silu_mul")(_p(gu), _p(out), c_int(T), c_int(I2 // 2), c_int(_DT[gu.dtype])), "silu_mul")
    return out


def qkv_prepare(qkv: torch.Tensor, k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], wq, wk, inv_freq,
                rotary_dim: int, eps: float, positions, seq_of_token, block_table, nh: int, nkv: int, hd: int) -> torch.Tensor:
    """Returns the prepared queries ``[T, nh * hd]``; writes keys and values into the pages."""
    T = qkv.shape[0]
    q_out = torch.empty((T, nh * hd), dtype=qkv.dtype)
    positions, seq_of_token, block_table = _i32(positions), _i32(seq_of_token), _i32(block_table)
    n_pages = (k_pages if k_pages is not None else v_pages).shape[0] if (k_pages is not None or v_pages is not None) else 0
    _check(_fn("sx_ref_qkv_prepare")(_p(qkv), _p(q_out), _p(k_pages), _p(v_pages), _p(wq), _p(wk), _p(inv_freq),
                                     c_int(rotary_dim), c_float(eps), _p(positions), _p(seq_of_token), _p(block_table),
                                     c_int(block_table.shape[1]), c_int(T), c_int(nh), c_int(nkv), c_int(hd), c_int(n_pages),
                                     c_int(_DT[qkv.dtype])), "qkv_prepare")
    return q_out


def attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, positions, seq_of_token, block_table, nh: int,
              nkv: int, hd: int, scale: float, window: Optional[int]) -> torch.Tensor:
    T = q.shape[0]
    out = torch.empty((T, nh * hd), dtype=q.dtype)
    positions, seq_of_token, block_table = _i32(positions), _i32(seq_of_token), _i32(block_table)
    _check(_fn("sx_ref_attn")(_p(q), _p(k_pages), _p(v_pages), _p(out), _p(positions), _p(seq_of_token), _p(block_table),
                              c_int(block_table.shape[1]), c_int(T), c_int(nh), c_int(nkv), c_int(hd), c_float(scale),
                              c_int(window or 0), c_int(_DT[q.dtype])), "attention")
    return out


def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    R, V = logits.shape
    out = torch.empty(R, dtype=torch.int32)
    _check(_fn("sx_ref_argmax_rows")(_p(logits), _p(out), c_int(R), c_int(V)), "argmax_rows")
    return out


def apply_penalties(logits: torch.Tensor, hist: torch.Tensor, hist_len: torch.Tensor, last_n: int, repetition: float,
                    presence: float, frequency: float) -> None:
    R, V = logits.shape
    hist, hist_len = _i32(hist), _i32(hist_len)
    _check(_fn("sx_ref_penalties")(_p(logits), _p(hist), _p(hist_len), c_int(hist.shape[1]), c_int(last_n), c_float(repetition),
                                   c_float(presence), c_float(frequency), c_int(R), c_int(V)), "penalties")


def sample_rows(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float, seed: int, seq_index,
                step, want_kept: bool = False):
    """``(tokens int32 [R], u float32 [R], kept uint8 [R, V] or None)``."""
    R, V = logits.shape
    seq_index, step = _i32(seq_index), _i32(step)
    out = torch.empty(R, dtype=torch.int32)
    u = torch.zeros(R, dtype=torch.float32)
    kept = torch.zeros((R, V), dtype=torch.uint8) if want_kept and temperature > 0 else None
    _check(_fn("sx_ref_sample_rows")(_p(logits), _p(out), c_int(R), c_int(V), c_float(temperature), c_int(top_k), c_float(top_p),
                                     c_float(min_p), ctypes.c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), _p(seq_index), _p(step),
                                     _p(u), _p(kept)), "sample_rows")
    return out, u, kept


def decode_begin(token_ids, control, history, hist_len) -> None:
    S = token_ids.numel()
    _check(_fn("sx_ref_decode_begin")(_p(token_ids), _p(control), _p(history), _p(hist_len),
                                      c_int(0 if history is None else history.shape[1]), c_int(S)), "decode_begin")


def decode_advance(token_ids, sampled, positions, seq_past, seq_lens, rng_step, advance_by, history, hist_len) -> None:
    S = token_ids.numel()
    _check(_fn("sx_ref_decode_advance")(_p(token_ids), _p(sampled), _p(positions), _p(seq_past), _p(seq_lens), _p(rng_step),
                                        _p(advance_by), _p(history), _p(hist_len),
                                        c_int(0 if history is None else history.shape[1]), c_int(S)), "decode_advance")
