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
from ..cache import PAGE_TOKENS, Cache, pages_for
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
    """Where each index array of a step lies in the one int32 buffer that is uploaded.

    ``decode=True`` is the layout of a decode session: the arrays that the device itself moves on
    after every step (tokens, positions, lengths, the random stream's step, the length of the
    penalties' history) come first, and everything from ``fixed_start`` on is written by the host
    alone, so it can be uploaded again (a sequence reached a new page) while steps are in flight.
    """
    MOVING = ("token_ids", "positions", "seq_past", "seq_lens", "rng_step", "hist_len")

    def __init__(self, T: int, S: int, R: int, maxp: int, ngroups: int, decode: bool = False):
        self.T, self.S, self.R, self.maxp, self.ngroups = T, S, R, maxp, ngroups
        if decode:
            arrays = [("token_ids", T), ("positions", T), ("seq_past", S), ("seq_lens", S), ("rng_step", S),
                      ("hist_len", S), ("seq_of_token", T), ("cu_seqlens", S + 1), ("seq_slots", S),
                      ("want_rows", R), ("advance_by", S), ("request", S)]
        else:
            arrays = [("token_ids", T), ("positions", T), ("seq_of_token", T), ("cu_seqlens", S + 1),
                      ("seq_past", S), ("seq_lens", S), ("seq_slots", S), ("want_rows", R)]
        arrays += [(("block_table", g), S * maxp) for g in range(ngroups)]
        self.where = {}
        off = 0
        self.fixed_start = 0
        for name, size in arrays:
            if decode and name == "seq_of_token":
                self.fixed_start = off
            self.where[name] = (off, size)
            off += _align4(size)
        self.total = off

    def views(self, flat):
        """name -> view of ``flat`` (numpy or torch), block tables as a list under 'block_tables'."""
        out = {n: flat[o:o + z] for n, (o, z) in self.where.items() if isinstance(n, str)}
        out["block_tables"] = [
            flat[self.where[("block_table", g)][0]:self.where[("block_table", g)][0] + self.S * self.maxp].reshape(
                self.S, self.maxp) for g in range(self.ngroups)]
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
        """Copy ``flat`` to the device (into ``into[:len(flat)]`` if given), asynchronously."""
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
        ev = self.events[i]
        if ev is None:
            ev = self.events[i] = torch.cuda.Event()
        ev.record()
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


class _Captured:
    """Single-token steps of ``S`` rows with block tables ``maxp`` pages wide, with their index
    arrays at fixed addresses: ``body()`` is run eagerly the first time and replayed as a CUDA
    graph afterwards (or run eagerly every time when the engine does not use graphs)."""

    def __init__(self, engine: "Engine", S: int, maxp: int, decode: bool = False):
        self.engine = engine
        self.layout = _Layout(S, S, S, maxp, engine.cache.n_block_tables, decode=decode)
        self.flat = torch.zeros(self.layout.total, dtype=torch.int32, device=engine.device)
        self.arrays = v = self.layout.views(self.flat)
        self.ctx = StepContext(
            token_ids=v["token_ids"], positions=v["positions"], seq_of_token=v["seq_of_token"],
            cu_seqlens=v["cu_seqlens"], seq_past=v["seq_past"], seq_lens=v["seq_lens"], seq_slots=v["seq_slots"],
            want_rows=v["want_rows"], block_tables=v["block_tables"], n_tokens=S, n_seqs=S, n_want=S, max_new=1,
            max_len=maxp * PAGE_TOKENS, all_single=True, runtime=engine.runtime, want_all=True)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.result: Optional[torch.Tensor] = None
        self.launches = 0
        self.in_use = False

    def body(self) -> torch.Tensor:
        return self.engine._forward(self.ctx)

    def run(self) -> torch.Tensor:
        eng = self.engine
        if self.graph is not None:
            self.graph.replay()
            eng.kernel_launches += self.launches
            return self.result
        before = eng.kernel_launches
        out = self.body()                               # eager: the real result of this step
        self.launches = eng.kernel_launches - before
        if eng.use_graphs:
            g = torch.cuda.CUDAGraph()
            with _capture(g):                           # recorded, not run: nothing is touched
                self.result = self.body()
            eng.kernel_launches = before + self.launches
            self.graph = g
        return out


class _CapturedDecode(_Captured):
    """A captured step that also samples and moves on, all on the device: the model, the sampler
    (``params``), and the advance of tokens, positions, lengths and the random stream's step.

    ``control [S]`` is written by the host before every step: ``-1`` lets a row take the token the
    device sampled for it in the step before, any other value is the token the row runs instead.
    ``sampled [S]`` holds the step's tokens afterwards.  ``history [S, hist_cap]`` (only when
    ``params`` has penalties) is each row's context, which the advance appends to.
    """

    def __init__(self, engine: "Engine", S: int, maxp: int, params):
        super().__init__(engine, S, maxp, decode=True)
        self.params = params
        dev = engine.device
        self.control = torch.full((S,), -1, dtype=torch.int32, device=dev)
        self.sampled = torch.zeros(S, dtype=torch.int32, device=dev)
        self.hist_cap = maxp * PAGE_TOKENS + 1 if params.penalties_on else 0
        self.history = torch.zeros((S, self.hist_cap), dtype=torch.int32, device=dev) if self.hist_cap else None

    def body(self) -> torch.Tensor:
        from ..sampling.sampler import sample_on_device
        a = self.arrays
        ops.decode_begin(a["token_ids"], self.control)
        logits = self.engine._forward(self.ctx)
        sample_on_device(self.params, logits, a["request"], a["rng_step"], self.history, a["hist_len"],
                         out=self.sampled)
        ops.decode_advance(a["token_ids"], self.sampled, a["positions"], a["seq_past"], a["seq_lens"],
                           a["rng_step"], a["advance_by"], self.history, a["hist_len"])
        return self.sampled


class DecodeRow(NamedTuple):
    """One sequence of a decode session: its slot, the token it runs next, and what the sampler
    needs: the request's index and how many tokens it has sampled so far (they pick the word of
    its random stream), and its context (prompt and output so far) if penalties are on."""
    slot: int
    token: int
    request: int = 0
    sampled_so_far: int = 0
    context: Optional[Sequence[int]] = None


class Engine:
    """A loaded model with its cache: slots are opened, stepped and closed here."""

    def __init__(self, model, *, max_tokens: int, max_seqs: Optional[int] = None, use_graphs: bool = True,
                 nvtx: bool = False):
        """``nvtx``: name every step for a profiler's timeline (NVTX ranges ``prompt step`` / ``decode step`` with
        the number of sequences and tokens), as the reference's telemetry does
        (crates/synaptix-runtime/src/telemetry/nvtx.rs); off by default, it costs two calls a step."""
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
        self.nvtx = bool(nvtx)
        self._captured: Dict[Tuple[int, int], _Captured] = {}
        self._captured_decode: Dict[tuple, _CapturedDecode] = {}
        self.kernel_launches = 0         # kernels of this package launched (graph replays counted by content)
        ops.set_launch_counter(self)

    @property
    def max_tokens(self) -> int:
        return self.cache.max_tokens

    @property
    def max_seqs(self) -> int:
        return self.cache.max_seqs

    @property
    def free_tokens(self) -> int:
        """Tokens the pages hold that no open sequence has: what new sequences can still take."""
        return min(pool.n_free for pool in self.cache.slots.pools) * PAGE_TOKENS

    @property
    def free_seqs(self) -> int:
        return self.cache.max_seqs - self.cache.slots.n_live

    @property
    def h2d_bytes(self) -> int:
        """Bytes of step index arrays uploaded from pinned host memory so far."""
        return self._staging.bytes_uploaded

    # -- slots -----------------------------------------------------------------
    def open(self) -> int:
        return self.cache.open()

    def close(self, slot: int) -> None:
        self.cache.close(slot)

    def length(self, slot: int) -> int:
        return self.cache.slots.length(slot)

    @contextlib.contextmanager
    def _range(self, name: str):
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()

    def check_kernels(self) -> None:
        """Raise ``KernelError`` if a bounded wait inside one of the tensor-memory kernels ran out
        since the last call (their results are then not to be trusted).  Costs no device call."""
        ops.check_status()

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
        # dummy rows: token 0 at position 0 of page 0, which no sequence owns, in the state row no sequence owns
        spare = self.cache.spare_slot
        for i in range(len(entries), lay.S):
            sot[t0] = i
            cu[i] = t0
            v["seq_lens"][i] = 1
            v["seq_slots"][i] = spare
            v["want_rows"][r0] = t0
            r0 += 1
            t0 += 1
        cu[lay.S] = t0
        self._fill_tables(v, [e.slot for e in entries], lay.maxp)
        return flat

    def _fill_tables(self, v, slot_ids: Sequence[int], maxp: int) -> None:
        slots = self.cache.slots
        for g, bt in enumerate(v["block_tables"]):
            for i, s in enumerate(slot_ids):
                row = np.asarray(slots.table(s, g)[:maxp], dtype=np.int32)
                bt[i, :row.shape[0]] = np.maximum(row, 0)       # pages given back (-1) read as page 0

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
        (a caller that samples from it at once needs no copy)."""
        entries = [e if isinstance(e, Entry) else Entry(*e) for e in entries]
        past, new = self._check(entries)
        single = all(n == 1 and tuple(e.want) == (0,) for n, e in zip(new, entries))
        if not self.nvtx:
            return self._run_step(entries, past, new, single, keep)
        with self._range(f"{'decode' if max(new) == 1 else 'prompt'} step: {len(entries)} sequences, {sum(new)} tokens"):
            return self._run_step(entries, past, new, single, keep)

    def _run_step(self, entries, past, new, single, keep) -> torch.Tensor:
        if single and self.use_graphs:
            S = _bucket_rows(len(entries))
            maxp = _bucket_pages(max(pages_for(p + 1) for p in past))
            cap = self._captured.get((S, maxp))
            if cap is None:
                cap = self._captured[(S, maxp)] = _Captured(self, S, maxp)
            flat = self._fill(cap.layout, entries, past, new)
            self._staging.upload(flat, into=cap.flat)
            logits = cap.run()[:len(entries)]
            if keep:
                logits = logits.clone()
        else:
            ctx = self.plan(entries, past, new)
            logits = self._forward(ctx)
        for e in entries:
            self.cache.slots.advance(e.slot, len(e.tokens))
        return logits

    # -- decoding -------------------------------------------------------------------
    def start_decode(self, rows: Sequence[DecodeRow], sampling=None) -> "DecodeSession":
        """A decode session for sequences that have run their prompts: see ``DecodeSession``."""
        return DecodeSession(self, rows, sampling)


class _Pending:
    """A launched step whose tokens the host has not handed out yet."""
    __slots__ = ("buf", "event", "n", "tokens")

    def __init__(self, buf, event, n):
        self.buf, self.event, self.n, self.tokens = buf, event, n, None

    def read(self) -> List[int]:
        if self.tokens is None:
            self.event.synchronize()
            self.tokens = self.buf[:self.n].tolist()
        return self.tokens


class DecodeSession:
    """Single-token steps of a set of sequences, with sampling and the move to the next token
    kept on the device: a step's sampled tokens are the next step's input without passing
    through the host.  The host only enqueues (``launch``) and reads tokens as they arrive
    (``collect``), so it can enqueue step k+1 before it has seen the tokens of step k.

    ``launch()`` reserves the cache pages the step needs (``CacheFull`` leaves everything as it
    was), writes the step's control words (and, when a sequence reached a new page, its page
    tables) and enqueues the step: one CUDA graph of model, sampler and advance once it has been
    recorded.  ``collect()`` waits for the oldest step not yet read and returns its tokens, one per
    live row.  ``drop(rows)`` takes sequences out; all launched steps must have been collected.
    What a step computes is what ``Engine.step`` computes for the same tokens: both run the
    model through ``Engine._forward`` on the same cache.

    A generation loop that sees a stop token in step k's tokens has usually launched step k+1
    already; that step then ran one token too many for the stopped row, into pages the row still
    held, and its token for that row is dropped.  The reference's loop has the same shape without
    the lookahead (crates/synaptix-models/llm/qwen3/src/pipeline.rs:279-302: graph replay, the
    sampled token copied back each step).
    """

    def __init__(self, engine: Engine, rows: Sequence[DecodeRow], sampling=None):
        from ..sampling.params import SamplingParams
        self.engine = engine
        self.params = sampling if sampling is not None else SamplingParams()
        self.params.validate()
        self.rows: List[DecodeRow] = []
        self.lens: List[int] = []             # tokens each row holds after the steps launched so far
        self.sampled: List[int] = []          # tokens each row has sampled, launched steps included
        self.last: List[Optional[int]] = []   # the token each row runs next, if the host knows it
        self.contexts: List[Optional[List[int]]] = []
        self.pending: List[_Pending] = []
        self.cap: Optional[_CapturedDecode] = None
        self._stale = True                    # the device arrays must be written anew before the next step
        self._tables: List[tuple] = []
        self._free: List[tuple] = []          # (pinned buffer, event) pairs not in use
        self.d2h_bytes = 0
        vocab = engine.model.embedding.vocab
        seen = set()
        for r in rows:
            r = r if isinstance(r, DecodeRow) else DecodeRow(*r)
            if r.slot in seen:
                raise StepError(f"slot {r.slot} appears twice in one decode session")
            seen.add(r.slot)
            if not (0 <= r.token < vocab):
                raise StepError(f"slot {r.slot}: token ids must lie in [0, {vocab})")
            if self.params.penalties_on and r.context is None:
                raise StepError("penalties need each row's context")
            self.rows.append(r)
            self.lens.append(engine.cache.slots.length(r.slot))
            self.sampled.append(r.sampled_so_far)
            self.last.append(int(r.token))
            self.contexts.append(list(r.context) if r.context is not None else None)
        if not self.rows:
            raise StepError("a decode session needs at least one row")

    # -- state ------------------------------------------------------------------------
    @property
    def in_flight(self) -> int:
        return len(self.pending)

    @property
    def n_rows(self) -> int:
        return len(self.rows)

    def _release(self) -> None:
        if self.cap is not None:
            self.cap.in_use = False
            self.cap = None

    def close(self) -> None:
        """Give the captured step back to the engine (``drop`` of the last rows does it too)."""
        self._read_all()
        self._release()

    def _read_all(self) -> None:
        """Wait for every launched step and keep its tokens for ``collect``; afterwards the host
        knows the token each row runs next."""
        for p in self.pending:
            p.read()
        if self.pending:
            self.last = list(self.pending[-1].tokens)

    def _table_lens(self) -> List[tuple]:
        slots = self.engine.cache.slots
        return [slots.table_shape(r.slot) for r in self.rows]

    def _acquire(self, S: int, maxp: int) -> _CapturedDecode:
        eng = self.engine
        key = (S, maxp, self.params)
        cap = eng._captured_decode.get(key)
        if cap is None:
            cap = eng._captured_decode[key] = _CapturedDecode(eng, S, maxp, self.params)
        elif cap.in_use:                       # another session is on it: one of our own, not kept
            cap = _CapturedDecode(eng, S, maxp, self.params)
        cap.in_use = True
        return cap

    def _write_all(self, S: int, maxp: int) -> None:
        """Everything the device holds of this session, from what the host knows."""
        eng = self.engine
        self._read_all()
        if self.cap is None or (self.cap.layout.S, self.cap.layout.maxp) != (S, maxp):
            self._release()
            self.cap = self._acquire(S, maxp)
        cap = self.cap
        n = len(self.rows)
        # a step of one token each for the live rows, dummy rows behind them
        entries = [Entry(r.slot, [t], [0]) for r, t in zip(self.rows, self.last)]
        flat = eng._fill(cap.layout, entries, self.lens, [1] * n)
        v = cap.layout.views(flat)
        v["advance_by"][:n] = 1
        v["request"][:n] = [r.request for r in self.rows]
        v["rng_step"][:n] = self.sampled
        if cap.history is not None:
            hist = np.zeros((cap.layout.S, cap.hist_cap), dtype=np.int32)
            for i, c in enumerate(self.contexts):
                c = c + [p.tokens[i] for p in self.pending]        # launched steps the caller has not collected
                m = min(len(c), cap.hist_cap)
                hist[i, :m] = c[len(c) - m:]
                v["hist_len"][i] = m
            cap.history.copy_(torch.from_numpy(hist).pin_memory(), non_blocking=True)
            eng._staging.bytes_uploaded += hist.size * 4
        eng._staging.upload(flat, into=cap.flat)
        if not eng.use_graphs:
            cap.ctx.host = {"cu_seqlens": list(range(n + 1)), "seq_slots": [r.slot for r in self.rows]}
        self._tables = self._table_lens()
        self._stale = False

    def _write_tables(self) -> None:
        """The host-owned part of the device arrays again (page tables changed); the arrays the
        device moves on by itself are left alone, so steps may be in flight."""
        eng, cap = self.engine, self.cap
        lay = cap.layout
        n = len(self.rows)
        entries = [Entry(r.slot, [0], [0]) for r in self.rows]
        flat = eng._fill(lay, entries, self.lens, [1] * n)
        v = lay.views(flat)
        v["advance_by"][:n] = 1
        v["request"][:n] = [r.request for r in self.rows]
        eng._staging.upload(flat[lay.fixed_start:], into=cap.flat[lay.fixed_start:])
        self._tables = self._table_lens()

    # -- steps -------------------------------------------------------------------------
    def launch(self, tokens: Optional[Sequence[Optional[int]]] = None) -> None:
        """Enqueue one step.  ``tokens[i]``, if given and not ``None``, is the token row ``i`` runs
        in this step instead of the one sampled for it in the step before."""
        eng = self.engine
        slots = eng.cache.slots
        n = len(self.rows)
        if n == 0:
            raise StepError("the decode session has no rows left")
        vocab = eng.model.embedding.vocab
        if tokens is not None:
            if len(tokens) != n:
                raise StepError(f"{len(tokens)} tokens for {n} rows")
            for t in tokens:
                if t is not None and not (0 <= t < vocab):
                    raise StepError(f"token ids must lie in [0, {vocab})")
            if self.params.penalties_on:
                if self.pending:
                    raise StepError("with penalties on, tokens are put in only when no step is in flight")
                for c, t in zip(self.contexts, tokens):
                    if t is not None:
                        c[-1] = int(t)
        for r, ln in zip(self.rows, self.lens):
            if slots.length(r.slot) != ln:
                raise StepError(f"slot {r.slot} was stepped outside its decode session")
        slots.reserve_many([r.slot for r in self.rows], [1] * n)          # CacheFull: nothing has changed
        need_p = max(pages_for(ln + 1) for ln in self.lens)
        # a captured step has dummy rows up to a bucket; an eager one runs the live rows alone, since
        # parts that loop over sequences on the host see exactly those
        S = _bucket_rows(n) if eng.use_graphs else n
        cap = self.cap
        if self._stale or cap is None or cap.layout.S != S or cap.layout.maxp < need_p:
            self._write_all(S, _bucket_pages(need_p))
            cap = self.cap
        elif self._table_lens() != self._tables:
            self._write_tables()
        if not eng.use_graphs:              # parts that loop on the host get this step's lengths
            cap.ctx.host.update(seq_past=list(self.lens), seq_lens=[ln + 1 for ln in self.lens])
            cap.ctx.max_len = max(self.lens) + 1
        # control words: -1, or the token the host puts in
        ctl = np.full(cap.layout.S, -1, dtype=np.int32)
        if tokens is not None:
            for i, t in enumerate(tokens):
                if t is not None:
                    ctl[i] = t
        eng._staging.upload(ctl, into=cap.control)
        if eng.nvtx:
            with eng._range(f"decode step: {n} sequences"):
                cap.run()
        else:
            cap.run()
        buf, event = self._free.pop() if self._free else (
            torch.empty(max(eng.max_seqs, 64), dtype=torch.int32, pin_memory=True), torch.cuda.Event())
        buf[:n].copy_(cap.sampled[:n], non_blocking=True)
        event.record()
        self.pending.append(_Pending(buf, event, n))
        self.d2h_bytes += 4 * n
        for i, r in enumerate(self.rows):
            slots.advance(r.slot, 1)
            self.lens[i] += 1
            self.sampled[i] += 1
        self.last = [None] * n

    def collect(self) -> List[int]:
        """The tokens of the oldest launched step not yet collected, one per row."""
        if not self.pending:
            raise StepError("no step is in flight")
        p = self.pending.pop(0)
        tokens = p.read()
        if not self.pending:
            self.last = list(tokens)
        self._free.append((p.buf, p.event))
        if self.contexts and self.contexts[0] is not None:
            for c, t in zip(self.contexts, tokens):
                c.append(t)
        self.engine.check_kernels()
        return tokens

    def drop(self, rows: Sequence[int]) -> None:
        """Rows (indices into the live rows) leave the session; their slots are the caller's to close."""
        if self.pending:
            raise StepError("collect every launched step before rows are dropped")
        gone = set(rows)
        keep = [i for i in range(len(self.rows)) if i not in gone]
        for name in ("rows", "lens", "sampled", "last", "contexts"):
            old = getattr(self, name)
            setattr(self, name, [old[i] for i in keep])
        self._stale = True
        if not self.rows:
            self._release()
