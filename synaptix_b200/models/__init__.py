"""Models: from a typed configuration to parts, and from a folder to a loaded model."""
from __future__ import annotations

import torch

from ..config.registry import load_config, resolve_architecture
from ..parts.base import Runtime
from ..weights.loader import SafetensorsSource, WeightSource
from . import qwen3 as _qwen3  # registers the architecture
from .decoder import DecoderModel, LayerRun

__all__ = ["DecoderModel", "LayerRun", "model_skeleton", "load_model", "parse_dtype"]


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name in (torch.bfloat16, torch.float32):
            return name
        raise ValueError(f"compute dtype must be bfloat16 or float32, not {name}")
    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
             "fp32": torch.float32, "f32": torch.float32}
    try:
        return table[str(name).lower()]
    except KeyError:
        raise ValueError(f"compute dtype must be one of {sorted(table)}, not {name!r}") from None


def model_skeleton(config) -> DecoderModel:
    """The model of ``config``'s architecture with no weights bound (names and shapes only)."""
    entry = resolve_architecture({"architectures": list(type(config).architectures)})
    return entry.build(config)


def load_model(model_dir: str, dtype="bfloat16", device="cuda:0", source: WeightSource = None) -> DecoderModel:
    """Read ``config.json``, choose the model class by it, bind ``model.safetensors`` by name."""
    config = load_config(model_dir)
    model = model_skeleton(config)
    rt = Runtime(torch.device(device), parse_dtype(dtype))
    if source is None:
        source = SafetensorsSource(model_dir)
    return model.load(source, rt, where=f"weights in {model_dir}")
