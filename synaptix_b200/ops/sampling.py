"""Python faces of the sampling kernels in ``csrc/sampling.cu``."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import KernelError, c_float, c_int, c_ulonglong, check, fn, ptr, require_cuda, stream


def _rows(logits: torch.Tensor):
    require_cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise KernelError("sampling takes float32 logits [rows, vocab]")
    return logits.shape


def argmax_rows(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """int32 ``[rows]``: index of each row's maximum (the last one among equals).  Wide rows are
    cut into chunks scanned by blocks of their own, with a small second kernel to finish."""
    R, V = _rows(logits)
    if out is None:
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
    if V >= 16384:
        chunks = min(64, (V + 4095) // 4096)
        sv = torch.empty(R * chunks, dtype=torch.float32, device=logits.device)
        si = torch.empty(R * chunks, dtype=torch.int32, device=logits.device)
        check(fn("sampling", "sx_argmax_rows_chunked")(ptr(logits), ptr(out), ptr(sv), ptr(si), c_int(R), c_int(V),
                                                       c_int(chunks), stream()), "argmax_rows", launches=2)
        return out
    check(fn("sampling", "sx_argmax_rows")(ptr(logits), ptr(out), c_int(R), c_int(V), stream()), "argmax_rows")
    return out


def apply_penalties(logits: torch.Tensor, hist: torch.Tensor, hist_len: torch.Tensor, last_n: int,
                    repetition: float, presence: float, frequency: float) -> None:
    """In place: repetition, presence and frequency penalties over the last ``last_n`` tokens
    (0 = all) of each row's context ``hist[r, :hist_len[r]]``."""
    R, V = _rows(logits)
    require_cuda(hist, hist_len)
    if hist.dtype != torch.int32 or hist_len.dtype != torch.int32 or hist.shape[0] != R:
        raise KernelError("penalties: hist int32 [rows, n], hist_len int32 [rows]")
    counts = torch.zeros((R, V), dtype=torch.int32, device=logits.device)     # the kernel wants zeros and leaves zeros
    check(fn("sampling", "sx_penalties")(ptr(logits), ptr(counts), ptr(hist), ptr(hist_len), c_int(hist.shape[1]),
                                         c_int(last_n), c_float(repetition), c_float(presence),
                                         c_float(frequency), c_int(R), c_int(V), stream()), "penalties")


def sample_rows(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float,
                seed: int, seq_index: torch.Tensor, step: torch.Tensor,
                out: Optional[torch.Tensor] = None, u_out: Optional[torch.Tensor] = None,
                cluster: Optional[int] = None) -> torch.Tensor:
    """int32 ``[rows]``: argmax if ``temperature <= 0``; else temperature, top-k, top-p, min-p
    and a multinomial draw with the Philox word (``seed``, ``seq_index[r]``, ``step[r]``).

    ``cluster``: None lets the library choose between its two kernels by the row's width (one block a row, or a
    row spread over a cluster of blocks); 0 asks for the one-block kernel, 1, 2, 4 or 8 for that many blocks a row."""
    R, V = _rows(logits)
    require_cuda(seq_index, step, out, u_out)
    if seq_index.dtype != torch.int32 or step.dtype != torch.int32:
        raise KernelError("sample_rows: seq_index and step are int32")
    if out is None:
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
    if cluster:
        check(fn("sampling", "sx_sample_rows_cluster")(ptr(logits), ptr(out), c_int(R), c_int(V), c_float(temperature),
                                                       c_int(top_k), c_float(top_p), c_float(min_p),
                                                       c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), ptr(seq_index),
                                                       ptr(step), ptr(u_out), c_int(cluster), stream()),
              "sample_rows")
        return out
    if cluster == 0:
        check(fn("sampling", "sx_sample_rows_block")(ptr(logits), ptr(out), c_int(R), c_int(V), c_float(temperature),
                                                     c_int(top_k), c_float(top_p), c_float(min_p),
                                                     c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), ptr(seq_index),
                                                     ptr(step), ptr(u_out), stream()), "sample_rows")
        return out
    check(fn("sampling", "sx_sample_rows")(ptr(logits), ptr(out), c_int(R), c_int(V), c_float(temperature),
                                           c_int(top_k), c_float(top_p), c_float(min_p),
                                           c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), ptr(seq_index), ptr(step),
                                           ptr(u_out), stream()), "sample_rows")
    return out
