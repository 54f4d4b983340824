"""Random-weights mode: weights drawn from a configuration and a seed.

Nothing like it exists in the reference for whole models (every WeightSource
there is file-backed); the nearest is ``init_tensor(shape, Normal{mean,std},
dtype, seed)`` (crates/synaptix-nn/src/init.rs:20-47).  Each tensor has a random
stream of its own, keyed by the seed and the tensor's NAME, so that a tensor's
values do not depend on which other tensors exist or in which order they are
drawn.

``RandomSource`` serves tensors straight to a model (on any device, which is
how the benchmark avoids writing gigabytes to disk); ``write_model_folder``
writes ``config.json`` and ``model.safetensors`` for a typed configuration.

One seed gives one set of values PER DEVICE KIND: torch's CPU and CUDA generators
draw different normal numbers from the same seed, so ``device="cuda:0"`` and
``device="cpu"`` give two different (equally valid) random models.  A model folder is
always written from the CPU generator, so the same seed writes the same bytes on any
machine; whoever needs an engine and an oracle to agree loads both from one folder.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Mapping, Optional, Tuple

import torch

from .loader import TensorSpec, WeightSource
from .safetensors_io import write_safetensors


def _stream_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


class RandomSource(WeightSource):
    """Seeded normal weights for a set of tensor specs.

    ``matrix`` ~ N(0, std_matrix), ``embedding`` ~ N(0, std_embedding),
    ``gain`` ~ 1 + N(0, std_gain), ``table`` = zeros (int32).  Floating tensors
    are drawn in float32 and stored as ``dtype`` (``gain_dtype`` for gains).
    """

    def __init__(self, specs: Mapping[str, TensorSpec], seed: int, *,
                 std_matrix: float = 0.02, std_embedding: Optional[float] = None,
                 std_gain: float = 0.05, dtype: torch.dtype = torch.bfloat16,
                 gain_dtype: Optional[torch.dtype] = None, device: str = "cpu",
                 skip_optional: bool = True):
        self.specs = {n: s for n, s in specs.items() if not (s.optional and skip_optional)}
        self.seed = int(seed)
        self.std_matrix = float(std_matrix)
        self.std_embedding = float(std_matrix if std_embedding is None else std_embedding)
        self.std_gain = float(std_gain)
        self.dtype = dtype
        self.gain_dtype = dtype if gain_dtype is None else gain_dtype
        self.device = torch.device(device)

    def shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {n: tuple(s.shape) for n, s in self.specs.items()}

    def get(self, name: str) -> torch.Tensor:
        spec = self.specs[name]
        if spec.kind == "table":
            return torch.zeros(spec.shape, dtype=torch.int32, device=self.device)
        g = torch.Generator(device=self.device)
        g.manual_seed(_stream_seed(self.seed, name))
        x = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=self.device)
        if spec.kind == "gain":
            return (1.0 + self.std_gain * x).to(self.gain_dtype)
        if spec.kind == "embedding":
            return (self.std_embedding * x).to(self.dtype)
        if spec.kind == "matrix":
            return (self.std_matrix * x).to(self.dtype)
        raise ValueError(f"tensor {name!r}: unknown kind {spec.kind!r}")


def write_model_folder(config, out_dir: str, seed: int, **random_kwargs) -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors`` for ``config``.

    The tensor names and shapes are the ones the architecture's model asks for;
    ``random_kwargs`` go to ``RandomSource`` (standard deviations, dtypes).
    """
    from ..models import model_skeleton  # late: models import parts import weights

    model = model_skeleton(config)
    specs = model.all_tensor_specs()
    src = RandomSource(specs, seed, device="cpu", **random_kwargs)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=2)
        f.write("\n")
    tensors = {n: src.get(n) for n in src.shapes()}
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return out_dir
