"""A decoder model as data: parts, and the order in which layers run.

``layers`` are blocks; ``schedule`` lists the runs of a step in order.  A run
names a layer and the cache entry it works on, so a schedule may run a layer
twice (two runs, each with a cache entry of its own) or let a layer read the
cache another layer wrote (``write_cache=False`` and that layer's entry).  The
default schedule runs every layer once on its own entry.

Step (crates/synaptix-models/llm/common/src/model.rs:1057-1117,1160-1262):
embedding -> runs -> final norm on the rows whose logits are wanted -> output
head.  The reference normalises all rows and then narrows (model.rs:1068-1074);
here only the wanted rows are normalised and projected.
"""
from __future__ import annotations

import dataclasses
import weakref
from typing import Dict, List, Mapping, Optional, Sequence

import torch

from .. import ops
from ..cache.store import CacheRequest
from ..ops.decode_stream import enabled as stream_enabled
from ..parts.base import Norm, Part, PendingLinear, Runtime, StepContext, plain
from ..parts.embedding import Embedding, OutputHead
from ..weights.loader import TensorSpec, WeightSource, bind_tensors


@dataclasses.dataclass(frozen=True)
class LayerRun:
    layer: int
    cache_entry: int
    write_cache: bool = True


class DecoderModel(Part):
    def __init__(self, config, embedding: Embedding, layers: Sequence[Part], final_norm: Norm,
                 head: OutputHead, schedule: Optional[Sequence[LayerRun]] = None,
                 stop_token_ids: Sequence[int] = ()):
        self.config = config
        self.embedding = embedding
        self.layers = list(layers)
        self.final_norm = final_norm
        self.head = head
        self.schedule = list(schedule) if schedule is not None else [
            LayerRun(i, i) for i in range(len(self.layers))]
        self.stop_token_ids = tuple(stop_token_ids)
        self.runtime: Optional[Runtime] = None
        self._stream_cache: dict = {}
        n_entries = 1 + max((r.cache_entry for r in self.schedule), default=-1)
        owners: List[Optional[int]] = [None] * n_entries
        for r in self.schedule:
            if not (0 <= r.layer < len(self.layers)):
                raise ValueError(f"schedule names layer {r.layer}, the model has {len(self.layers)}")
            if r.write_cache:
                if owners[r.cache_entry] is not None:
                    raise ValueError(f"cache entry {r.cache_entry} is written by two runs")
                owners[r.cache_entry] = r.layer
        for r in self.schedule:
            if owners[r.cache_entry] is None:
                raise ValueError(f"cache entry {r.cache_entry} is read but never written")
        self._entry_owner = owners

    @property
    def vocab_size(self) -> int:
        return self.head.vocab

    def children(self) -> List[Part]:
        return [self.embedding] + self.layers + [self.final_norm, self.head]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def cache_requests(self) -> List[CacheRequest]:
        """One request per cache entry, asked of the layer that writes it."""
        return [self.layers[o].cache_request() for o in self._entry_owner]

    # -- weights -----------------------------------------------------------
    def load(self, source: WeightSource, rt: Runtime, where: str = "weights") -> "DecoderModel":
        tensors = bind_tensors(self.all_tensor_specs(), source, where=where)
        self.bind_all(tensors, rt)
        self.runtime = rt
        return self

    # -- fused runs of layers ------------------------------------------------
    def _stream_segments(self, cache):
        """The schedule cut into pieces: ``(first run, last run + 1, plan)`` where ``plan`` is a
        ``StreamPlan`` over consecutive runs whose blocks offer themselves to the fused layer
        kernel with equal sizes, or ``None`` for runs that go through ``forward`` one by one.
        Built once per cache (the plan holds the addresses of its pages)."""
        key = id(cache)
        hit = self._stream_cache.get(key)
        if hit is not None and hit[0]() is cache:
            return hit[1]
        from ..ops.decode_stream import StreamPlan
        fields = [self.layers[r.layer].stream_fields(cache.view(r.cache_entry), r.write_cache)
                  for r in self.schedule]
        sizes = [None if f is None else (f["H"], f["nh"], f["nkv"], f["hd"], f["I"]) for f in fields]
        segments, i = [], 0
        while i < len(fields):
            j = i + 1
            if fields[i] is not None:
                while j < len(fields) and sizes[j] == sizes[i]:
                    j += 1
                plan = StreamPlan.build(fields[i:j], self.runtime.device)
            else:
                while j < len(fields) and fields[j] is None:
                    j += 1
                plan = None
            segments.append((i, j, plan))
            i = j
        self._stream_cache = {key: (weakref.ref(cache), segments)}
        return segments

    def stream_status(self) -> int:
        """0, or the first non-zero status word of the fused layer kernels (a bounded wait ran out)."""
        for _, (_, segments) in self._stream_cache.items():
            for _, _, plan in segments:
                if plan is not None and plan.status():
                    return plan.status()
        return 0

    # -- one step ------------------------------------------------------------
    def forward(self, ctx: StepContext, cache) -> torch.Tensor:
        """Logits float32 ``[n_want, vocab]`` for ``ctx.want_rows``."""
        h = self.embedding.forward(ctx.token_ids)
        pending = None
        fused = (ctx.all_single and 0 < ctx.n_tokens <= 8 and self.runtime is not None
                 and self.runtime.dtype == torch.bfloat16 and h.dtype == torch.float32 and stream_enabled())
        segments = self._stream_segments(cache) if fused else [(0, len(self.schedule), None)]
        for first, last, plan in segments:
            if plan is not None:
                if pending is not None:
                    ops.residual_add(h, plain(pending))
                    pending = None
                plan.run(h, ctx.positions, ctx.seq_lens, ctx.block_tables, ctx.max_len)
                continue
            for run in self.schedule[first:last]:
                if isinstance(pending, PendingLinear) and not getattr(self.layers[run.layer], "takes_pending_product", False):
                    pending = pending.materialize()
                h, pending = self.layers[run.layer].forward(h, pending, ctx, cache.view(run.cache_entry),
                                                            run.write_cache)
        if isinstance(pending, PendingLinear) and not self.final_norm.takes_pending_product:
            pending = pending.materialize()
        if getattr(ctx, "want_all", False):        # every row, in order: no gather, and the norm may fuse
            x = self.final_norm.add_forward(h, pending, lazy=True)
        else:
            x = self.final_norm.add_forward(h, pending, rows=ctx.want_rows)
        return self.head.forward(x)
