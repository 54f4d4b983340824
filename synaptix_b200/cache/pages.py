"""Bookkeeping of the cache: pages, and a slot for each live sequence.

The reference's model cache has ONE length for the whole batch
(crates/synaptix-models/llm/common/src/model.rs:349-368) and contiguous
``[B, n_kv, capacity, head_dim]`` storage per layer, so rows must advance
together.  Here every sequence has a slot with its own length, and storage is
handed out in pages of ``PAGE_TOKENS`` tokens, so that the cache is sized by
the number of tokens that live sequences hold, not by slots x capacity.

Nothing in this file touches a device: it is the part that must never lose a
page, hand one out twice or take one back twice, and it is tested on the CPU.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

PAGE_TOKENS = 64


class CacheFull(RuntimeError):
    """No free page (or slot) is left for what a step needs."""


class SlotError(RuntimeError):
    """A slot or page was used after it was given back, given back twice, or never handed out."""


def pages_for(tokens: int) -> int:
    return (tokens + PAGE_TOKENS - 1) // PAGE_TOKENS


class PagePool:
    """A free list over page ids ``first .. first+n_pages-1``.

    Pages are handed out lowest-id-first from a stack, so a page that was just
    freed is the next one reused: reuse bugs show at once in tests.
    """

    def __init__(self, n_pages: int, first: int = 0):
        if n_pages < 0:
            raise ValueError("n_pages must be >= 0")
        self.n_pages = n_pages
        self.first = first
        self._free: List[int] = list(range(first + n_pages - 1, first - 1, -1))
        self._held = [False] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> List[int]:
        """``n`` pages, or ``CacheFull`` with nothing taken."""
        if n > len(self._free):
            raise CacheFull(f"cache is full: {n} more pages of {PAGE_TOKENS} tokens wanted, "
                            f"{len(self._free)} of {self.n_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p - self.first] = True
        return out

    def free(self, pages: Sequence[int]) -> None:
        for p in pages:
            i = p - self.first
            if not (0 <= i < self.n_pages):
                raise SlotError(f"page {p} does not belong to this pool")
            if not self._held[i]:
                raise SlotError(f"page {p} freed twice (or never handed out)")
        if len(set(pages)) != len(pages):
            raise SlotError("the same page is named twice in one free")
        for p in pages:
            self._held[p - self.first] = False
            self._free.append(p)

    def held(self) -> List[int]:
        return [self.first + i for i, h in enumerate(self._held) if h]


class GroupPages:
    """The pages one sequence holds in one storage group.

    ``table[i]`` is the page of tokens ``[i*PAGE_TOKENS, (i+1)*PAGE_TOKENS)``, or
    ``-1`` once a windowed group has let go of it.
    """
    __slots__ = ("table", "released")

    def __init__(self):
        self.table: List[int] = []
        self.released = 0      # leading entries already given back


class SequenceSlots:
    """Slots of live sequences over one ``PagePool`` per storage group.

    ``windows[g]`` is ``None`` for a group that keeps every key, or the number
    of latest keys a windowed group needs; a windowed group gives pages back as
    soon as no later query can see them.
    """

    def __init__(self, max_seqs: int, pools: Sequence[PagePool],
                 windows: Optional[Sequence[Optional[int]]] = None):
        self.max_seqs = max_seqs
        self.pools = list(pools)
        self.windows = list(windows) if windows is not None else [None] * len(self.pools)
        if len(self.windows) != len(self.pools):
            raise ValueError("one window entry per pool")
        self._free_slots: List[int] = list(range(max_seqs - 1, -1, -1))
        self._len: Dict[int, int] = {}
        self._pages: Dict[int, List[GroupPages]] = {}

    # -- slots ---------------------------------------------------------
    @property
    def n_live(self) -> int:
        return len(self._len)

    def live(self) -> List[int]:
        return sorted(self._len)

    def open(self) -> int:
        if not self._free_slots:
            raise CacheFull(f"all {self.max_seqs} sequence slots are in use")
        s = self._free_slots.pop()
        self._len[s] = 0
        self._pages[s] = [GroupPages() for _ in self.pools]
        return s

    def _check(self, slot: int) -> None:
        if slot not in self._len:
            raise SlotError(f"slot {slot} is not open")

    def close(self, slot: int) -> None:
        self._check(slot)
        for pool, gp in zip(self.pools, self._pages[slot]):
            pool.free([p for p in gp.table if p >= 0])
        del self._len[slot]
        del self._pages[slot]
        self._free_slots.append(slot)

    # -- lengths and pages --------------------------------------------------
    def length(self, slot: int) -> int:
        self._check(slot)
        return self._len[slot]

    def table(self, slot: int, group: int) -> List[int]:
        self._check(slot)
        return self._pages[slot][group].table

    def table_shape(self, slot: int) -> tuple:
        """Per group ``(pages in the table, leading pages given back)``: it changes exactly when
        the slot's page tables do."""
        self._check(slot)
        return tuple((len(gp.table), gp.released) for gp in self._pages[slot])

    def reserve(self, slot: int, n_new: int) -> None:
        """Make sure pages exist for ``n_new`` more tokens; on ``CacheFull`` nothing changes."""
        self._check(slot)
        if n_new < 0:
            raise ValueError("n_new must be >= 0")
        need = pages_for(self._len[slot] + n_new)
        wants = [max(0, need - len(gp.table)) for gp in self._pages[slot]]
        for pool, w in zip(self.pools, wants):
            if w > pool.n_free:
                raise CacheFull(f"cache is full: {w} more pages of {PAGE_TOKENS} tokens wanted, "
                                f"{pool.n_free} of {pool.n_pages} free")
        for pool, gp, w in zip(self.pools, self._pages[slot], wants):
            gp.table.extend(pool.alloc(w))

    def reserve_many(self, slots: Sequence[int], n_new: Sequence[int]) -> None:
        """``reserve`` for a whole batch, all or nothing."""
        per_pool = [0] * len(self.pools)
        for s, n in zip(slots, n_new):
            self._check(s)
            need = pages_for(self._len[s] + n)
            for g, gp in enumerate(self._pages[s]):
                per_pool[g] += max(0, need - len(gp.table))
        for pool, w in zip(self.pools, per_pool):
            if w > pool.n_free:
                raise CacheFull(f"cache is full: {w} more pages of {PAGE_TOKENS} tokens wanted, "
                                f"{pool.n_free} of {pool.n_pages} free")
        for s, n in zip(slots, n_new):
            self.reserve(s, n)

    def advance(self, slot: int, n: int) -> None:
        """The sequence now holds ``n`` more tokens (pages must have been reserved)."""
        self._check(slot)
        new_len = self._len[slot] + n
        for gp in self._pages[slot]:
            if pages_for(new_len) > len(gp.table):
                raise SlotError(f"slot {slot}: advanced to {new_len} tokens without reserved pages")
        self._len[slot] = new_len
        for pool, gp, w in zip(self.pools, self._pages[slot], self.windows):
            if w is None:
                continue
            # a later query sits at position >= new_len and sees keys > position - w,
            # so key j is dead once j <= new_len - w; page i holds keys up to i*P + P-1
            i = gp.released
            dead = []
            while i < len(gp.table) and i * PAGE_TOKENS + PAGE_TOKENS - 1 <= new_len - w:
                if gp.table[i] >= 0:
                    dead.append(gp.table[i])
                    gp.table[i] = -1
                i += 1
            gp.released = i
            if dead:
                pool.free(dead)

    def tokens_held(self) -> int:
        """Tokens held by live sequences, each rounded up to whole pages."""
        return sum(pages_for(n) * PAGE_TOKENS for n in self._len.values())
