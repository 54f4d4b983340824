"""The step function: a batch of sequences, each with its next tokens, run as ONE batch.

``Engine.step(entries)`` takes, for each sequence, its slot, its next tokens and
the places among them whose logits are wanted.  The tokens of all sequences are
packed into one stream; every token-parallel kernel runs on the packed stream,
attention and the cache write use each token's sequence and position, and the
final norm and output head run only on the wanted rows.  It runs only the
tokens it is given, from the cache earlier steps left, and returns float32
logits ``[n_wanted, vocab]`` in the order of the entries and of ``want``.
Prompts are never padded.  A step of single tokens may be replayed as a CUDA
graph captured for a fixed number of rows; rows beyond the live ones then run a
dummy token that writes to a cache page no sequence owns, and their logits are
dropped, so this padding changes no result either.

The reference's nearest equivalents are rectangular: ``DecoderModel::forward``
with one shared past length (crates/synaptix-models/llm/common/src/model.rs:
1052-1055,1107-1117) and ``forward_decode_dev`` for B rows of one token with
per-row positions, replayed as a CUDA graph
(:1489-1549; crates/synaptix-infer/src/graph_capture/capture.rs:24-122).
"""
from __future__ import annotations

import contextlib
import gc
from typing import Dict, List, NamedTuple, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
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


@contextlib.contextmanager
def _capture(graph: "torch.cuda.CUDAGraph"):
    """Stream capture with Python's cyclic garbage collector held off.  If the collector ran in the
    middle of a capture and freed an engine dropped earlier (its graphs and their memory pools), the
    driver calls made by those destructors would invalidate the capture."""
    was_on = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph):
            yield
    finally:
        if was_on:
            gc.enable()


class _Layout:
    """Where each index array of a step lies in the one int32 buffer that is uploaded."""
    NAMES = ("token_ids", "positions", "seq_of_token", "cu_seqlens", "seq_past", "seq_lens", "seq_slots",
             "want_rows")

    def __init__(self, T: int, S: int, R: int, maxp: int, ngroups: int):
        self.T, self.S, self.R, self.maxp, self.ngroups = T, S, R, maxp, ngroups
        sizes = [T, T, T, S + 1, S, S, S, R] + [S * maxp] * ngroups
        self.sizes = sizes
        self.offs = [0]
        for s in sizes:
            self.offs.append(self.offs[-1] + _align4(s))
        self.total = self.offs[-1]

    def views(self, flat):
        """name -> view of ``flat`` (numpy or torch), block tables as a list under 'block_tables'."""
        out = {n: flat[self.offs[i]:self.offs[i] + self.sizes[i]] for i, n in enumerate(self.NAMES)}
        out["block_tables"] = [
            flat[self.offs[8 + g]:self.offs[8 + g] + self.S * self.maxp].reshape(self.S, self.maxp)
            for g in range(self.ngroups)]
        return out


class _Staging:
    """Pinned host buffers for a step's index arrays, reused round-robin; a buffer is
    written again only after the copy that last read it has finished."""

    def __init__(self, device: torch.device, depth: int = 4):
        self.device = device
        self.bufs: List[Optional[torch.Tensor]] = [None] * depth
        self.events: List[Optional[torch.cuda.Event]] = [None] * depth
        self.i = 0
        self.bytes_uploaded = 0

    def upload(self, flat: np.ndarray, into: Optional[torch.Tensor] = None) -> torch.Tensor:
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
        dev = into if into is not None else torch.empty(n, dtype=torch.int32, device=self.device)
        dev[:n].copy_(buf[:n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        self.bytes_uploaded += n * 4
        return dev


def _bucket_rows(n: int) -> int:
    """Rows of a captured single-token step: 1, 2, 4, 8, then multiples of 8 up to 64, of 32 beyond."""
    if n <= 8:
        b = 1
        while b < n:
            b *= 2
        return b
    if n <= 64:
        return (n + 7) // 8 * 8
    return (n + 31) // 32 * 32


def _bucket_pages(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


class _CapturedStep:
    """A single-token step of ``S`` rows with block tables ``maxp`` pages wide, with its index
    arrays at fixed addresses, run eagerly the first time and replayed as a graph afterwards."""

    def __init__(self, engine: "Engine", S: int, maxp: int):
        self.engine = engine
        self.layout = _Layout(S, S, S, maxp, engine.cache.n_block_tables)
        self.flat = torch.zeros(self.layout.total, dtype=torch.int32, device=engine.device)
        v = self.layout.views(self.flat)
        self.ctx = StepContext(
            token_ids=v["token_ids"], positions=v["positions"], seq_of_token=v["seq_of_token"],
            cu_seqlens=v["cu_seqlens"], seq_past=v["seq_past"], seq_lens=v["seq_lens"], seq_slots=v["seq_slots"],
            want_rows=v["want_rows"], block_tables=v["block_tables"], n_tokens=S, n_seqs=S, n_want=S, max_new=1,
            max_len=maxp * PAGE_TOKENS, all_single=True, runtime=engine.runtime, want_all=True)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.launches = 0

    def run(self) -> torch.Tensor:
        eng = self.engine
        if self.graph is not None:
            self.graph.replay()
            eng.kernel_launches += self.launches
            return self.logits
        before = eng.kernel_launches
        out = eng._forward(self.ctx)                    # eager: the real result of this step
        self.launches = eng.kernel_launches - before
        g = torch.cuda.CUDAGraph()
        with _capture(g):                               # recorded, not run: the cache is untouched
            self.logits = eng._forward(self.ctx)
        eng.kernel_launches = before + self.launches
        self.graph = g
        return out


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
        self.use_graphs = bool(use_graphs) and model.all_graph_safe()
        self._captured: Dict[Tuple[int, int], _CapturedStep] = {}
        self._last_decode = None
        self.kernel_launches = 0         # kernels of this package launched (graph replays counted by content)
        ops.set_launch_counter(self)

    @property
    def max_tokens(self) -> int:
        return self.cache.max_tokens

    @property
    def max_seqs(self) -> int:
        return self.cache.max_seqs

    @property
    def h2d_bytes(self) -> int:
        """Bytes of step index arrays uploaded from pinned host memory so far."""
        return self._staging.bytes_uploaded

    # -- slots -----------------------------------------------------------------
    def open(self) -> int:
        return self.cache.open()

    def close(self, slot: int) -> None:
        self._last_decode = None
        self.cache.close(slot)

    def length(self, slot: int) -> int:
        return self.cache.slots.length(slot)

    # -- a step ------------------------------------------------------------------
    def _forward(self, ctx: StepContext) -> torch.Tensor:
        ops.set_launch_counter(self)
        return self.model.forward(ctx, self.cache)

    def _check(self, entries: Sequence[Entry]) -> Tuple[List[int], List[int]]:
        slots = self.cache.slots
        vocab = self.model.embedding.vocab
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"slot {e.slot}: an entry brings at least one token")
            slots.length(e.slot)            # raises SlotError if the slot is not open
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= vocab:
                raise StepError(f"slot {e.slot}: token ids must lie in [0, {vocab})")
            for w in e.want:
                if not (0 <= w < n):
                    raise StepError(f"slot {e.slot}: wanted place {w} is outside its {n} tokens")
        new = [len(e.tokens) for e in entries]
        slots.reserve_many([e.slot for e in entries], new)
        past = [slots.length(e.slot) for e in entries]
        return past, new

    def _fill(self, lay: _Layout, entries: Sequence[Entry], past: List[int], new: List[int]) -> np.ndarray:
        """The step's index arrays; rows of ``lay`` beyond the entries are dummy single tokens."""
        slots = self.cache.slots
        flat = np.zeros(lay.total, dtype=np.int32)
        v = lay.views(flat)
        tok, pos, sot, cu = v["token_ids"], v["positions"], v["seq_of_token"], v["cu_seqlens"]
        t0 = r0 = 0
        for i, e in enumerate(entries):
            n = new[i]
            tok[t0:t0 + n] = e.tokens
            pos[t0:t0 + n] = np.arange(past[i], past[i] + n)
            sot[t0:t0 + n] = i
            cu[i] = t0
            v["seq_past"][i] = past[i]
            v["seq_lens"][i] = past[i] + n
            v["seq_slots"][i] = e.slot
            for w in e.want:
                v["want_rows"][r0] = t0 + w
                r0 += 1
            t0 += n
        for i in range(len(entries), lay.S):          # dummy rows: token 0 at position 0 of the unowned page 0
            sot[t0] = i
            cu[i] = t0
            v["seq_lens"][i] = 1
            v["seq_slots"][i] = 0
            v["want_rows"][r0] = t0
            r0 += 1
            t0 += 1
        cu[lay.S] = t0
        for g in range(lay.ngroups):
            bt = v["block_tables"][g]
            for i, e in enumerate(entries):
                row = np.asarray(slots.table(e.slot, g)[:lay.maxp], dtype=np.int32)
                bt[i, :row.shape[0]] = np.maximum(row, 0)
        return flat

    def plan(self, entries: Sequence[Entry], past: List[int], new: List[int]) -> StepContext:
        """Upload the step's index arrays and wrap them."""
        S, T = len(entries), sum(new)
        R = sum(len(e.want) for e in entries)
        maxp = max(pages_for(p + n) for p, n in zip(past, new))
        lay = _Layout(T, S, R, maxp, self.cache.n_block_tables)
        flat = self._fill(lay, entries, past, new)
        v = lay.views(self._staging.upload(flat))
        return StepContext(
            token_ids=v["token_ids"], positions=v["positions"], seq_of_token=v["seq_of_token"],
            cu_seqlens=v["cu_seqlens"], seq_past=v["seq_past"], seq_lens=v["seq_lens"], seq_slots=v["seq_slots"],
            want_rows=v["want_rows"], block_tables=v["block_tables"],
            n_tokens=T, n_seqs=S, n_want=R, max_new=max(new), max_len=max(p + n for p, n in zip(past, new)),
            all_single=all(n == 1 for n in new), runtime=self.runtime,
            want_all=(R == T and all(tuple(e.want) == tuple(range(len(e.tokens))) for e in entries)),
            host={"cu_seqlens": lay.views(flat)["cu_seqlens"].tolist(), "seq_past": list(past),
                  "seq_lens": [p + n for p, n in zip(past, new)], "seq_slots": [e.slot for e in entries]})

    def step(self, entries: Sequence[Entry], keep: bool = True) -> torch.Tensor:
        """Run one step; returns float32 logits ``[n_wanted, vocab]`` on the device.

        With ``keep=False`` the result may be a buffer that the next step overwrites
        (the generation loop samples from it at once and needs no copy)."""
        entries = [e if isinstance(e, Entry) else Entry(*e) for e in entries]
        if self.use_graphs:
            logits = self._step_again(entries)
            if logits is not None:
                return logits.clone() if keep else logits
        past, new = self._check(entries)
        single = all(n == 1 and tuple(e.want) == (0,) for n, e in zip(new, entries))
        if single and self.use_graphs:
            S = _bucket_rows(len(entries))
            maxp = _bucket_pages(max(pages_for(p + 1) for p in past))
            cap = self._captured.get((S, maxp))
            if cap is None:
                cap = self._captured[(S, maxp)] = _CapturedStep(self, S, maxp)
            flat = self._fill(cap.layout, entries, past, new)
            self._staging.upload(flat, into=cap.flat)
            logits = cap.run()[:len(entries)]
            # remembered for the next step of the same sequences (see _step_again)
            self._last_decode = (tuple(e.slot for e in entries), [p + 1 for p in past], cap, flat)
            if keep:
                logits = logits.clone()
        else:
            self._last_decode = None
            ctx = self.plan(entries, past, new)
            logits = self._forward(ctx)
        for e in entries:
            self.cache.slots.advance(e.slot, len(e.tokens))
        return logits

    def _step_again(self, entries: Sequence[Entry]) -> Optional[torch.Tensor]:
        """The common case of decoding: the same sequences as in the last step, one more token
        each, and nobody crosses into a new page.  Then the index arrays of the last step are
        still right but for the tokens and the positions, which move on by one: no planning."""
        last = self._last_decode
        if last is None:
            return None
        key, lens, cap, flat = last
        n = len(entries)
        if n != len(key):
            return None
        vocab = self.model.embedding.vocab
        slots = self.cache.slots
        toks = []
        for e, s, ln in zip(entries, key, lens):
            if e.slot != s or len(e.tokens) != 1 or tuple(e.want) != (0,) or ln % PAGE_TOKENS == 0:
                return None
            t = e.tokens[0]
            if not (0 <= t < vocab) or slots._len.get(s) != ln:
                return None
            toks.append(t)
        v = cap.layout.views(flat)
        v["token_ids"][:n] = toks
        v["positions"][:n] += 1
        v["seq_past"][:n] += 1
        v["seq_lens"][:n] += 1
        self._staging.upload(flat, into=cap.flat)
        logits = cap.run()[:n]
        for i, s in enumerate(key):
            slots.advance(s, 1)
            lens[i] += 1
        return logits

    # -- decoding without coming back to the host ------------------------------------
    def decode_run(self, slots: Sequence[int], tokens: Sequence[int], n_steps: int, sampler=None) -> torch.Tensor:
        """``n_steps`` single-token steps for ``slots`` starting from ``tokens``, each step's
        sampled token fed to the next on the device; returns the sampled tokens int32
        ``[n_steps, len(slots)]`` (on the device).  See ``DecodeRun``."""
        if n_steps <= 0:
            return torch.empty((0, len(slots)), dtype=torch.int32, device=self.device)
        return DecodeRun(self, slots, tokens, n_steps, sampler).steps(n_steps)


class DecodeRun:
    """Single-token steps of a fixed set of sequences that never come back to the host: each
    step's sampled token is the next step's input, positions advance on the device, and the
    whole step (model, sampling, advance) is one CUDA graph after its first, eager run.

    Pages for ``max_steps`` more tokens are reserved up front, so block tables do not change.
    ``sampler(logits) -> int32 [rows]`` runs on the device inside the step (default: argmax).
    Stop tokens are not looked at; the generation loop is the place for that.
    """

    def __init__(self, engine: Engine, slots: Sequence[int], tokens: Sequence[int], max_steps: int, sampler=None):
        from ..ops import sampling as K
        self.engine = engine
        self.slots = list(slots)
        self.max_steps = max_steps
        self.done = 0
        entries = [Entry(s, [t], [0]) for s, t in zip(slots, tokens)]
        past, _ = engine._check(entries)
        engine.cache.slots.reserve_many(self.slots, [max_steps] * len(self.slots))
        S = len(entries)
        maxp = max(pages_for(p + max_steps) for p in past)
        lay = _Layout(S, S, S, maxp, engine.cache.n_block_tables)
        flat = engine._staging.upload(engine._fill(lay, entries, past, [1] * S)).clone()
        v = lay.views(flat)
        self.ctx = ctx = StepContext(
            token_ids=v["token_ids"], positions=v["positions"], seq_of_token=v["seq_of_token"],
            cu_seqlens=v["cu_seqlens"], seq_past=v["seq_past"], seq_lens=v["seq_lens"], seq_slots=v["seq_slots"],
            want_rows=v["want_rows"], block_tables=v["block_tables"], n_tokens=S, n_seqs=S, n_want=S, max_new=1,
            max_len=maxp * PAGE_TOKENS, all_single=True, runtime=engine.runtime, want_all=True)
        self.sampled = sampled = torch.empty(S, dtype=torch.int32, device=engine.device)

        def one():
            logits = engine._forward(ctx)
            tok = K.argmax_rows(logits, out=sampled) if sampler is None else sampler(logits)
            if tok is not sampled:
                sampled.copy_(tok)
            ops.decode_advance(ctx.token_ids, sampled, ctx.positions, ctx.seq_past, ctx.seq_lens)

        self._one = one
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches_per_step = 0

    def steps(self, n: int) -> torch.Tensor:
        """Run ``n`` more steps; returns their sampled tokens int32 ``[n, rows]`` on the device."""
        eng = self.engine
        if self.done + n > self.max_steps:
            raise StepError(f"this run reserved {self.max_steps} steps, {self.done} are done, {n} more asked")
        out = torch.empty((n, len(self.slots)), dtype=torch.int32, device=eng.device)
        for k in range(n):
            if self.graph is None:
                before = eng.kernel_launches
                self._one()                                   # eager: the real step
                self.launches_per_step = eng.kernel_launches - before
                if eng.use_graphs:
                    g = torch.cuda.CUDAGraph()
                    with _capture(g):
                        self._one()                           # recorded, not run
                    eng.kernel_launches = before + self.launches_per_step
                    self.graph = g
            elif self.graph is not None:
                self.graph.replay()
                eng.kernel_launches += self.launches_per_step
            out[k].copy_(self.sampled)
        self.done += n
        for s in self.slots:
            eng.cache.slots.advance(s, n)
        return out
