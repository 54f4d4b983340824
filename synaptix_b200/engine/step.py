"""The step function: a batch of sequences, each with its next tokens, run as ONE batch.

``Engine.step(entries)`` takes, for each sequence, its slot, its next tokens and
the places among them whose logits are wanted.  The tokens of all sequences are
packed into one stream; every token-parallel kernel runs on the packed stream,
attention and the cache write use each token's sequence and position, and the
final norm and output head run only on the wanted rows.  It runs only the
tokens it is given, from the cache earlier steps left, and returns float32
logits ``[n_wanted, vocab]`` in the order of the entries and of ``want``.
There is no padding, so padding cannot change a result.

The reference's nearest equivalents are rectangular: ``DecoderModel::forward``
with one shared past length (crates/synaptix-models/llm/common/src/model.rs:
1052-1055,1107-1117) and ``forward_decode_dev`` for B rows of one token with
per-row positions (:1489-1549).
"""
from __future__ import annotations

from typing import List, NamedTuple, Optional, Sequence

import numpy as np
import torch

from ..cache import PAGE_TOKENS, Cache, CacheFull, SlotError, pages_for
from ..csrc.build import KernelsUnavailable
from ..parts.base import StepContext


class Entry(NamedTuple):
    """One sequence's part of a step."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepError(ValueError):
    """A step that cannot be run as given (bad token id, bad index, empty entry)."""


def _align4(n: int) -> int:
    return (n + 3) & ~3


class _Staging:
    """Pinned host buffers for a step's index arrays, reused round-robin; a buffer is
    written again only after the copy that last read it has finished."""

    def __init__(self, device: torch.device, depth: int = 4):
        self.device = device
        self.bufs: List[Optional[torch.Tensor]] = [None] * depth
        self.events: List[Optional[torch.cuda.Event]] = [None] * depth
        self.i = 0

    def upload(self, flat: np.ndarray) -> torch.Tensor:
        n = flat.shape[0]
        i = self.i
        self.i = (i + 1) % len(self.bufs)
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.bufs[i]
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 4096), dtype=torch.int32, pin_memory=True)
            self.bufs[i] = buf
        buf[:n].numpy()[:] = flat
        dev = torch.empty(n, dtype=torch.int32, device=self.device)
        dev.copy_(buf[:n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        return dev


class Engine:
    """A loaded model with its cache: slots are opened, stepped and closed here."""

    def __init__(self, model, *, max_tokens: int, max_seqs: Optional[int] = None, use_graphs: bool = True):
        if model.runtime is None:
            raise ValueError("the model has no weights bound")
        rt = model.runtime
        if rt.device.type != "cuda" or not torch.cuda.is_available():
            raise KernelsUnavailable(
                "the engine runs only on a CUDA device (sm_100a); there is no CPU path")
        self.model = model
        self.runtime = rt
        self.device = rt.device
        self.cache = Cache(model.cache_requests(), max_tokens=max_tokens, max_seqs=max_seqs,
                           dtype=rt.dtype, device=rt.device)
        self._staging = _Staging(rt.device)
        self.use_graphs = use_graphs

    @property
    def max_tokens(self) -> int:
        return self.cache.max_tokens

    @property
    def max_seqs(self) -> int:
        return self.cache.max_seqs

    # -- slots -----------------------------------------------------------------
    def open(self) -> int:
        return self.cache.open()

    def close(self, slot: int) -> None:
        self.cache.close(slot)

    def length(self, slot: int) -> int:
        return self.cache.slots.length(slot)

    # -- a step ------------------------------------------------------------------
    def plan(self, entries: Sequence[Entry]) -> StepContext:
        """Check the entries, reserve pages and upload the step's index arrays."""
        slots = self.cache.slots
        vocab = self.model.embedding.vocab
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if len(e.tokens) == 0:
                raise StepError(f"slot {e.slot}: an entry brings at least one token")
            slots.length(e.slot)            # raises SlotError if the slot is not open
        new = [len(e.tokens) for e in entries]
        slots.reserve_many([e.slot for e in entries], new)

        S, T = len(entries), sum(new)
        past = [slots.length(e.slot) for e in entries]
        ngroups = self.cache.n_block_tables
        maxp = max(pages_for(p + n) for p, n in zip(past, new))
        R = sum(len(e.want) for e in entries)

        sizes = [T, T, T, S + 1, S, S, S, R] + [S * maxp] * ngroups
        offs = [0]
        for s in sizes:
            offs.append(offs[-1] + _align4(s))
        flat = np.zeros(offs[-1], dtype=np.int32)
        tok = flat[offs[0]:offs[0] + T]
        pos = flat[offs[1]:offs[1] + T]
        sot = flat[offs[2]:offs[2] + T]
        cu = flat[offs[3]:offs[3] + S + 1]
        sp = flat[offs[4]:offs[4] + S]
        sl = flat[offs[5]:offs[5] + S]
        ss = flat[offs[6]:offs[6] + S]
        wr = flat[offs[7]:offs[7] + R]
        t0 = 0
        r0 = 0
        for i, e in enumerate(entries):
            n = new[i]
            arr = np.asarray(e.tokens, dtype=np.int64)
            if arr.ndim != 1 or (arr < 0).any() or (arr >= vocab).any():
                raise StepError(f"slot {e.slot}: token ids must lie in [0, {vocab})")
            tok[t0:t0 + n] = arr
            pos[t0:t0 + n] = np.arange(past[i], past[i] + n)
            sot[t0:t0 + n] = i
            cu[i] = t0
            sp[i] = past[i]
            sl[i] = past[i] + n
            ss[i] = e.slot
            for w in e.want:
                if not (0 <= w < n):
                    raise StepError(f"slot {e.slot}: wanted place {w} is outside its {n} tokens")
                wr[r0] = t0 + w
                r0 += 1
            t0 += n
        cu[S] = T
        for g in range(ngroups):
            bt = flat[offs[8 + g]:offs[8 + g] + S * maxp].reshape(S, maxp)
            for i, e in enumerate(entries):
                tb = slots.table(e.slot, g)
                row = np.asarray(tb[:maxp], dtype=np.int32)
                bt[i, :row.shape[0]] = np.maximum(row, 0)

        dev = self._staging.upload(flat)

        def cut(k, n, shape=None):
            t = dev[offs[k]:offs[k] + n]
            return t if shape is None else t.view(shape)

        return StepContext(
            token_ids=cut(0, T), positions=cut(1, T), seq_of_token=cut(2, T), cu_seqlens=cut(3, S + 1),
            seq_past=cut(4, S), seq_lens=cut(5, S), seq_slots=cut(6, S), want_rows=cut(7, R),
            block_tables=[cut(8 + g, S * maxp, (S, maxp)) for g in range(ngroups)],
            n_tokens=T, n_seqs=S, n_want=R, max_new=max(new), max_len=max(p + n for p, n in zip(past, new)),
            all_single=all(n == 1 for n in new), runtime=self.runtime,
            host={"cu_seqlens": cu.tolist(), "seq_past": list(past), "seq_lens": [p + n for p, n in zip(past, new)],
                  "seq_slots": [e.slot for e in entries]})

    def step(self, entries: Sequence[Entry]) -> torch.Tensor:
        """Run one step; returns float32 logits ``[n_wanted, vocab]`` on the device."""
        entries = [e if isinstance(e, Entry) else Entry(*e) for e in entries]
        ctx = self.plan(entries)
        logits = self.model.forward(ctx, self.cache)
        for e in entries:
            self.cache.slots.advance(e.slot, len(e.tokens))
        return logits
