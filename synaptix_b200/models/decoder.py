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
from typing import Dict, List, Optional, Sequence

import torch

from ..cache.store import CacheRequest
from ..parts.base import Norm, Part, PendingLinear, Runtime, StepContext
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

    # -- one step ------------------------------------------------------------
    def forward(self, ctx: StepContext, cache) -> torch.Tensor:
        """Logits float32 ``[n_want, vocab]`` for ``ctx.want_rows``."""
        h = self.embedding.forward(ctx.token_ids)
        pending = None
        for run in self.schedule:
            if isinstance(pending, PendingLinear) and not getattr(self.layers[run.layer], "takes_pending_product", False):
                pending = pending.materialize()
            h, pending = self.layers[run.layer].forward(h, pending, ctx, cache.view(run.cache_entry), run.write_cache)
        if isinstance(pending, PendingLinear) and not self.final_norm.takes_pending_product:
            pending = pending.materialize()
        if getattr(ctx, "want_all", False):        # every row, in order: no gather, and the norm may fuse
            x = self.final_norm.add_forward(h, pending, lazy=True)
        else:
            x = self.final_norm.add_forward(h, pending, rows=ctx.want_rows)
        return self.head.forward(x)
