"""What every part of a layer is, and what a step hands to the parts.

A model is put together from parts; each part has its sizes and constants as
constructor parameters, names the tensors it needs, and is chosen by the
architecture's builder layer by layer.  No part knows which model it is in:
the tensor-name prefix it is given is data like any other.

Interfaces (a new part of any kind implements the one of its kind):

``Part``           ``tensor_specs() -> {name: TensorSpec}``; ``bind(tensors, runtime)``.
``Norm``           ``forward(h)`` and ``add_forward(h, delta, rows=None)``: ``h`` is the
                   float32 residual stream ``[T, width]``; ``add_forward`` first adds
                   ``delta`` into it; both return the normalised rows in the compute dtype
                   (or, with ``lazy=True``, a ``PendingNorm`` / ``ScaledRows`` that a product can finish).
``PositionEncoding`` ``rotation() -> (inv_freq float32 [rotary_dim/2], rotary_dim) | None``:
                   rotate-half rotation by ``position * inv_freq[i]``, applied to queries and
                   keys inside the fused head-preparation kernel.
``Mixer``          ``cache_request() -> KVRequest | StateRequest | None``;
                   ``forward(x, ctx, cache_view, write_cache=True) -> [T, width]``.
``FeedForward``    ``forward(x, ctx) -> [T, width]``.
``Block``          ``forward(h, pending, ctx, cache_view, write_cache) -> (h, pending)`` where
                   ``pending`` is a branch output not yet added into ``h`` (so that the sum can
                   be fused with the next norm).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Mapping, Optional

import torch

from ..weights.loader import TensorSpec


@dataclasses.dataclass
class Runtime:
    """Where and in which precision a model runs."""
    device: torch.device
    dtype: torch.dtype          # compute and cache dtype: torch.bfloat16 or torch.float32

    @property
    def is_fp32(self) -> bool:
        return self.dtype == torch.float32


class StepContext:
    """One step's batch, packed: the tokens of all sequences in one stream.

    Device tensors (int32): ``token_ids [T]``, ``positions [T]`` (absolute position of each
    token in its sequence), ``seq_of_token [T]`` (row of the per-sequence arrays),
    ``cu_seqlens [S+1]`` (first packed token of each sequence), ``seq_past [S]`` (tokens
    held before the step), ``seq_lens [S]`` (held after it), ``seq_slots [S]`` (cache slot),
    ``block_tables[g] [S, max_pages]`` (pages of each sequence in storage group ``g``),
    ``want_rows [R]`` (packed indices whose logits are wanted).

    Host values: ``n_tokens``, ``n_seqs``, ``n_want``, ``max_new`` (longest run of new
    tokens), ``max_len`` (longest sequence after the step), ``all_single`` (every sequence
    brings exactly one token), and ``host``: a dict of Python lists ``cu_seqlens``, ``seq_past``,
    ``seq_lens``, ``seq_slots`` for parts that loop over sequences on the host.  Inside a
    captured graph the host values are upper bounds and ``host`` is ``None``: a part that needs
    it sets ``graph_safe = False`` and the engine then runs every step eagerly.
    """
    __slots__ = ("token_ids", "positions", "seq_of_token", "cu_seqlens", "seq_past", "seq_lens",
                 "seq_slots", "block_tables", "want_rows", "n_tokens", "n_seqs", "n_want",
                 "max_new", "max_len", "all_single", "runtime", "scratch", "host", "want_all")

    def __init__(self, **kw):
        self.scratch = {}
        self.host = None
        self.want_all = False      # want_rows is 0..n_tokens-1 in order
        for k, v in kw.items():
            setattr(self, k, v)


class PendingNorm:
    """A normalised activation that has not been computed yet: ``rmsnorm(h + delta) * gain``.

    A norm may hand this to a consumer that says it can take it (``accepts_lazy_input``); a
    matrix product that can compute the norm in its own prologue then does so and writes the
    residual sum to ``h_out``, so the norm needs no kernel and no round trip through memory.
    Whoever cannot use it calls ``materialize()`` and gets the plain tensor.
    """
    __slots__ = ("h", "delta", "gain", "eps", "dtype", "_x", "_h_after")

    def __init__(self, h, delta, gain, eps, dtype):
        self.h, self.delta, self.gain, self.eps, self.dtype = h, delta, gain, eps, dtype
        self._x = None
        self._h_after = None

    @property
    def shape(self):
        return self.h.shape

    def h_out(self):
        """Where a fused consumer writes ``h + delta`` (``None`` when there is no delta)."""
        if self.delta is None:
            self._h_after = self.h
            return None
        if self._h_after is None or self._h_after is self.h:
            self._h_after = torch.empty_like(self.h)
        return self._h_after

    def materialize(self) -> torch.Tensor:
        if self._x is None:
            from .. import ops
            if self._h_after is not None and self._h_after is not self.h:
                # a fused consumer has already formed the sum; normalise that
                self._x = ops.add_rmsnorm(self._h_after, None, self.gain, self.eps, self.dtype)
            else:
                self._x = ops.add_rmsnorm(self.h, self.delta, self.gain, self.eps, self.dtype)
                self._h_after = self.h
        return self._x

    def h_after(self) -> torch.Tensor:
        """The residual stream after the sum, whoever formed it."""
        if self._h_after is None:
            self.materialize()
        return self._h_after


class PendingLinear:
    """A branch's last matrix product that has not run yet: ``x @ weight.T``.

    A mixer or feed-forward that is asked to (``forward(..., defer_output=True)``; only parts with
    ``can_defer_output`` are asked) may return this instead of the product.  A norm that says
    ``takes_pending_product`` may then run the product so that it adds itself into the residual stream and
    prepares the norm (``ScaledRows``); anybody else calls ``materialize()`` and gets the plain tensor.
    """
    __slots__ = ("x", "weight", "_y")

    def __init__(self, x, weight):
        self.x, self.weight = x, weight
        self._y = None

    @property
    def shape(self):
        return (self.x.shape[0], self.weight.shape[0])

    def materialize(self) -> torch.Tensor:
        if self._y is None:
            from .. import ops
            self._y = ops.linear(self.x, self.weight)
        return self._y


def plain(t):
    """``t`` as a tensor, whatever deferred form it came in."""
    return t.materialize() if isinstance(t, (PendingLinear, PendingNorm, ScaledRows)) else t


class ScaledRows:
    """A normalised activation that lacks its row factor: ``x = bf16(h * gain)`` and partial sums of squares
    ``ssq [T, n]`` of ``h``, so that ``rmsnorm(h) * gain = x * rsqrt(sum(ssq) / width + eps)``.  The product that
    formed the residual sum ``h`` made both on its way; a matrix product that takes this applies the factor to its
    results, so the norm costs no kernel.  ``materialize()`` gives the plain tensor (one norm kernel over ``h``)."""
    __slots__ = ("x", "ssq", "eps", "h", "gain", "dtype", "_plain")

    def __init__(self, x, ssq, eps, h, gain, dtype):
        self.x, self.ssq, self.eps, self.h, self.gain, self.dtype = x, ssq, eps, h, gain, dtype
        self._plain = None

    @property
    def shape(self):
        return self.x.shape

    def materialize(self) -> torch.Tensor:
        if self._plain is None:
            from .. import ops
            self._plain = ops.add_rmsnorm(self.h, None, self.gain, self.eps, self.dtype)
        return self._plain

    def h_after(self) -> torch.Tensor:
        return self.h


class Part:
    """Anything that owns tensors."""

    graph_safe = True      # False: forward depends on host values of the step (no CUDA graph)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        pass

    def children(self) -> List["Part"]:
        return []

    # helpers -------------------------------------------------------------
    def all_tensor_specs(self) -> Dict[str, TensorSpec]:
        out = dict(self.tensor_specs())
        for c in self.children():
            for n, s in c.all_tensor_specs().items():
                if n in out and out[n] != s:
                    raise ValueError(f"tensor {n!r} is asked for twice with different shapes")
                out[n] = s
        return out

    def all_graph_safe(self) -> bool:
        return self.graph_safe and all(c.all_graph_safe() for c in self.children())

    def bind_all(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.bind(tensors, rt)
        for c in self.children():
            c.bind_all(tensors, rt)


class Norm(Part):
    takes_pending_product = False  # True: add_forward may be handed a PendingLinear as delta

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_forward(self, h: torch.Tensor, delta: Optional[torch.Tensor],
                    rows: Optional[torch.Tensor] = None, lazy: bool = False):
        """``lazy=True`` allows the norm to return a ``PendingNorm`` (see there)."""
        raise NotImplementedError


class PositionEncoding(Part):
    def rotation(self):
        return None


class Mixer(Part):
    accepts_lazy_input = False     # True: forward may be handed a PendingNorm or ScaledRows instead of a tensor
    can_defer_output = False       # True: forward takes defer_output=True and may then return a PendingLinear

    def cache_request(self):
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache_view, write_cache: bool = True) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    accepts_lazy_input = False
    can_defer_output = False

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


def to_device_matrix(t: torch.Tensor, rt: Runtime) -> torch.Tensor:
    """A matrix in the compute dtype on the device (a 32-bit matrix is rounded once, to
    nearest even, when the compute dtype is bfloat16)."""
    return t.to(device=rt.device, dtype=rt.dtype).contiguous()


def to_device_f32(t: torch.Tensor, rt: Runtime) -> torch.Tensor:
    """A gain vector in 32-bit on the device (widening bfloat16 loses nothing)."""
    return t.to(device=rt.device, dtype=torch.float32).contiguous()
