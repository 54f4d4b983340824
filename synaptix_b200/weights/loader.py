"""Binding weights to a model by tensor name.

A model says which tensors it needs (name -> ``TensorSpec``); a source says
which it has.  ``bind_tensors`` compares the two completely before anything is
loaded and raises ONE ``WeightError`` listing every missing tensor, every
unexpected tensor and every wrong shape, so that a bad checkpoint is diagnosed
in a single run.  The reference reports only the first missing key
(crates/synaptix-models/llm/qwen3/src/loader.rs:118-128) and never checks shapes
against the config.

Storage dtype is kept: bfloat16 stays bfloat16 and a tensor stored in 32-bit
stays 32-bit; float16 is widened to float32 (lossless); integer tables come
back as int32.  What a part then does with its tensors (matrices go to the
compute dtype, norm gains stay in 32-bit) is the part's business.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, NamedTuple, Optional, Tuple

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile, resolve_shards


class TensorSpec(NamedTuple):
    """What a part expects of one tensor.

    ``kind`` steers the random-weights mode only: ``matrix`` and ``embedding``
    are zero-mean normal, ``gain`` is one plus normal, ``table`` is an integer
    table (filled with zeros).
    """
    shape: Tuple[int, ...]
    kind: str = "matrix"
    optional: bool = False


class WeightError(ValueError):
    """Weights do not fit the model: lists missing, unexpected and wrongly shaped tensors."""

    def __init__(self, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 other: Optional[List[str]] = None, where: str = "weights"):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.other = list(other or [])
        lines = [f"{where} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        for o in self.other:
            lines.append("  " + o)
        super().__init__("\n".join(lines))


class WeightSource:
    """Where tensors come from.  ``shapes()`` must be cheap (no data read)."""

    def shapes(self) -> Dict[str, Tuple[int, ...]]:
        raise NotImplementedError

    def get(self, name: str) -> torch.Tensor:
        """The tensor in its stored dtype (float16 widened, integers as int32), on the CPU
        unless the source creates tensors on a device."""
        raise NotImplementedError


def _normalise_dtype(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float32):
        return t
    if t.dtype in (torch.float16, torch.float64):
        return t.to(torch.float32)
    if t.dtype in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool):
        return t.to(torch.int32)
    raise WeightError([], [], [], [f"unsupported dtype {t.dtype}"])


class SafetensorsSource(WeightSource):
    """All shards of a model folder, indexed once (file discovery as in
    crates/synaptix-models/llm/qwen3/src/loader.rs:87-115)."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self._files = [SafetensorsFile(p) for p in resolve_shards(model_dir)]
        self._where: Dict[str, SafetensorsFile] = {}
        for f in self._files:
            for n in f.names():
                if n in self._where:
                    raise SafetensorsError(
                        f"tensor {n!r} appears in both {self._where[n].path} and {f.path}")
                self._where[n] = f

    def shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {n: f.tensors[n].shape for n, f in self._where.items()}

    def stored_dtype(self, name: str) -> str:
        return self._where[name].tensors[name].dtype

    def get(self, name: str) -> torch.Tensor:
        return _normalise_dtype(self._where[name].get(name))


class DictSource(WeightSource):
    """Tensors already in memory (tests, and models assembled by hand)."""

    def __init__(self, tensors: Mapping[str, torch.Tensor]):
        self._t = dict(tensors)

    def shapes(self):
        return {n: tuple(t.shape) for n, t in self._t.items()}

    def get(self, name):
        return _normalise_dtype(self._t[name])


def check_tensors(specs: Mapping[str, TensorSpec], shapes: Mapping[str, Tuple[int, ...]],
                  where: str = "weights") -> None:
    """Raise one ``WeightError`` naming everything that does not fit, or return."""
    missing = sorted(n for n, s in specs.items() if n not in shapes and not s.optional)
    unexpected = sorted(n for n in shapes if n not in specs)
    wrong = sorted((n, tuple(shapes[n]), tuple(s.shape)) for n, s in specs.items()
                   if n in shapes and tuple(shapes[n]) != tuple(s.shape))
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong, where=where)


def bind_tensors(specs: Mapping[str, TensorSpec], source: WeightSource,
                 where: str = "weights") -> Dict[str, torch.Tensor]:
    """Check ``source`` against ``specs`` as a whole, then fetch every tensor present."""
    shapes = source.shapes()
    check_tensors(specs, shapes, where=where)
    return {n: source.get(n) for n in specs if n in shapes}
