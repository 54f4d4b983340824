"""The generation loop above the step function.

For each batch: all prompts in one step (unequal lengths), one token sampled per
sequence from the logits at its last prompt token, then steps of one token for
every sequence still running.  A sequence ends when it emits a stop token (which
is part of its output), when it has ``max_new_tokens`` tokens (the first sampled
token counts), or when the cache cannot hold another token; its slot is given
back at once and the later steps shrink.  Requests beyond one batch run as
further batches, one after another, in the slots the earlier ones gave back.

The single-token steps run as a decode session of the engine: sampling and the move
to the next token stay on the device, the loop enqueues a step and reads the tokens of
the step before while it runs.  A stop token is therefore seen when the next step is
already on its way; that step's token for the stopped sequence is dropped (the
sequence ends with the stop token, exactly as without the lookahead), and a sequence
that ends by its length never runs a step too many, since the loop counts.

Single-sequence semantics follow the reference's loop
(crates/synaptix-models/llm/common/src/generate.rs:237-302: the stop check is on
the last emitted token before the next model call, :281-285; ``eos_set`` :202-208).
The loop knows the engine only as ``open() / close(slot) / step(entries) -> logits /
start_decode(rows, sampling) -> session`` (``launch``, ``collect``, ``drop``,
``in_flight``) and ``check_kernels()`` and the sampler of the prompt step only as a function of logits, so
its decisions are tested on the CPU with fakes of all of them.
"""
from __future__ import annotations

import dataclasses
import time
from typing import Callable, List, Optional, Sequence, Tuple

from ..cache.pages import PAGE_TOKENS, CacheFull, pages_for
from ..sampling.params import SamplingParams
from .step import DecodeRow, Entry


@dataclasses.dataclass(frozen=True)
class GenerationOptions:
    max_new_tokens: int = 64
    stop_token_ids: Tuple[int, ...] = ()
    sampling: SamplingParams = SamplingParams()
    max_batch_size: Optional[int] = None      # None: as many as the cache holds
    prefill_batch: int = 0                    # prompts run in portions of this many tokens a sequence (0: whole, in one step)
    lookahead: int = 2                        # decode steps enqueued before the oldest one's tokens are read


@dataclasses.dataclass
class GenerationResult:
    tokens: List[int]
    finish_reason: str          # "stop", "length", "capacity" or "cancelled" (the token callback returned False)
    prompt_tokens: int


@dataclasses.dataclass
class GenerationStats:
    """As the reference's GenerationStats (generate.rs:59-65), summed over batches."""
    prompt_tokens: int = 0
    new_tokens: int = 0
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    batches: int = 0
    decode_steps: int = 0
    decode_h2d_bytes: int = 0     # bytes of index arrays uploaded from pinned memory during decode steps
    decode_d2h_bytes: int = 0     # bytes of sampled tokens read back during decode steps


class _Live:
    __slots__ = ("request", "slot", "prompt", "out", "feed")

    def __init__(self, request, slot, prompt, cached=0):
        self.request, self.slot, self.prompt, self.out = request, slot, prompt, []
        self.feed = prompt[cached:] if cached else prompt       # what the prompt step runs: the cache holds the rest already


def plan_batches(prompt_lens: Sequence[int], max_new_tokens: int, max_tokens: int, max_seqs: int,
                 max_batch_size: Optional[int]) -> List[List[int]]:
    """Cut the request list, in order, into batches that fit the cache when every
    request runs to ``max_new_tokens`` (each request's tokens rounded up to whole pages).
    A request that does not fit even alone still gets a batch of its own if its prompt
    fits; it then ends by capacity."""
    total_pages = pages_for(max_tokens)
    limit = max_seqs if max_batch_size is None else min(max_seqs, max_batch_size)
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, n in enumerate(prompt_lens):
        if pages_for(n) > total_pages:
            raise CacheFull(f"request {i}: its prompt of {n} tokens does not fit a cache of "
                            f"{total_pages * PAGE_TOKENS} tokens")
        # the last sampled token is never fed back, so n + max_new - 1 tokens reach the cache
        need = min(pages_for(n + max(0, max_new_tokens - 1)), total_pages)
        if cur and (used + need > total_pages or len(cur) >= limit):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


def _run_prompts(engine, live, portion: int):
    """The prompts of a batch through the step function; returns the logits at every sequence's last prompt token,
    in the order of ``live``.  ``portion`` 0: all prompts whole, in one step.  Otherwise (the reference's
    ``prefill_batch``, generate.rs:255-271) in steps of at most ``portion`` tokens a sequence, which bounds a step's
    activations whatever the prompts' lengths; a sequence's logits come from the step that holds its last token."""
    if portion <= 0 or all(len(s.feed) <= portion for s in live):
        return engine.step([Entry(s.slot, s.feed, [len(s.feed) - 1]) for s in live], keep=False)
    rows = [None] * len(live)
    off = 0
    longest = max(len(s.feed) for s in live)
    while off < longest:
        part = [(i, s) for i, s in enumerate(live) if len(s.feed) > off]
        entries, ends = [], []
        for i, s in part:
            piece = s.feed[off:off + portion]
            last = off + len(piece) == len(s.feed)
            entries.append(Entry(s.slot, piece, [len(piece) - 1] if last else []))
            if last:
                ends.append(i)
        logits = engine.step(entries, keep=True)
        for k, i in enumerate(ends):
            rows[i] = logits[k]
        off += portion
    if hasattr(rows[0], "dim"):          # tensors from the engine (the loop's tests drive it with plain lists)
        import torch
        return torch.stack(rows)
    return rows


def run_generation(engine, sample: Callable, prompts: Sequence[Sequence[int]], options: GenerationOptions,
                   on_token: Optional[Callable[[int, int], None]] = None,
                   clock: Callable[[], float] = time.perf_counter, cached: Optional[Sequence[int]] = None):
    """Generate for every prompt; returns ``(results, stats)`` in the prompts' order.

    ``sample(logits, request_index, step, contexts) -> list of ints`` draws one token per row.
    ``on_token(request_index, token)`` is called for every token as it is produced.
    ``cached[i]``: so many leading tokens of prompt ``i`` are in the cache of the slot that ``engine.open()`` will
    return for it (a sequence that goes on from an earlier call, as the reference's ``generate_streaming_resume``
    starts its prompt at ``kv.seq_len``, generate.rs:248-250); the prompt step runs the rest, at least one token.
    """
    prompts = [list(p) for p in prompts]
    for i, p in enumerate(prompts):
        if not p:
            raise ValueError(f"request {i}: the prompt is empty")
        if cached is not None and not (0 <= cached[i] < len(p)):
            raise ValueError(f"request {i}: {cached[i]} cached tokens for a prompt of {len(p)}: at least one token must run")
    results: List[Optional[GenerationResult]] = [None] * len(prompts)
    stats = GenerationStats()
    if options.max_new_tokens <= 0:
        return [GenerationResult([], "length", len(p)) for p in prompts], stats
    stop = set(options.stop_token_ids)
    need_ctx = options.sampling.penalties_on

    def finish(seq: _Live, reason: str) -> None:
        engine.close(seq.slot)
        results[seq.request] = GenerationResult(seq.out, reason, len(seq.prompt))

    def take(seq: _Live, token: int) -> bool:
        """Record a token; True if the sequence goes on."""
        seq.out.append(token)
        stats.new_tokens += 1
        # (as the reference's StreamSink::on_token -> bool, generate.rs:67-75,279-291: a callback that returns False
        #  ends its sequence after this token; anything else, None included, lets it go on)
        if on_token is not None and on_token(seq.request, token) is False:
            finish(seq, "cancelled")
            return False
        if token in stop:
            finish(seq, "stop")
            return False
        if len(seq.out) >= options.max_new_tokens:
            finish(seq, "length")
            return False
        return True

    # what the cache can still take: all of it, unless sequences of other callers are open (a conversation beside this
    # call); a sequence that goes on brings its own pages along
    room_tokens = getattr(engine, "free_tokens", engine.max_tokens) if cached is None else engine.max_tokens
    room_seqs = getattr(engine, "free_seqs", engine.max_seqs) if cached is None else engine.max_seqs
    for batch in plan_batches([len(p) for p in prompts], options.max_new_tokens, room_tokens,
                              max(1, room_seqs), options.max_batch_size):
        stats.batches += 1
        live = [_Live(i, engine.open(), prompts[i], cached[i] if cached is not None else 0) for i in batch]
        t0 = clock()
        logits = _run_prompts(engine, live, options.prefill_batch)
        toks = sample(logits, [s.request for s in live], [0] * len(live),
                      [s.prompt for s in live] if need_ctx else None)
        engine.check_kernels()            # the host has waited for the prompt step: did all of it run?
        stats.prefill_ms += (clock() - t0) * 1e3
        stats.prompt_tokens += sum(len(s.feed) for s in live)
        live = [s for s, t in zip(live, toks) if take(s, int(t))]

        t0 = clock()
        up0 = getattr(engine, "h2d_bytes", 0)
        if live:
            session = engine.start_decode(
                [DecodeRow(s.slot, s.out[-1], s.request, len(s.out), (s.prompt + s.out) if need_ctx else None)
                 for s in live], options.sampling)
            depth = max(1, options.lookahead)
            full = False
            while live:       # (the session gives its captured step back when its last row is dropped)
                # all live sequences of a batch have the same number of tokens so far: they started together
                room = options.max_new_tokens - len(live[0].out) - session.in_flight
                if not full and room > 0 and session.in_flight < depth:
                    try:
                        session.launch()
                        stats.decode_steps += 1
                        continue
                    except CacheFull:
                        full = True
                if session.in_flight == 0:
                    # no page for everyone: the longest sequence ends, the others go on
                    victim = max(range(len(live)), key=lambda i: len(live[i].prompt) + len(live[i].out))
                    finish(live[victim], "capacity")
                    session.drop([victim])
                    del live[victim]
                    full = False
                    continue
                toks = session.collect()
                stats.decode_d2h_bytes += 4 * len(toks)
                gone = [i for i, (s, t) in enumerate(zip(live, toks)) if not take(s, int(t))]
                if gone:
                    # the steps already launched ran the ended sequences too; those tokens are dropped
                    while session.in_flight:
                        toks = session.collect()
                        stats.decode_d2h_bytes += 4 * len(toks)
                        for i, (s, t) in enumerate(zip(live, toks)):
                            if i not in gone and not take(s, int(t)):
                                gone.append(i)
                    session.drop(gone)
                    live = [s for i, s in enumerate(live) if i not in gone]
                full = False
        stats.decode_ms += (clock() - t0) * 1e3
        stats.decode_h2d_bytes += getattr(engine, "h2d_bytes", 0) - up0
    return results, stats
