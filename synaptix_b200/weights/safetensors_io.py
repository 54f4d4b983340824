"""Reader and writer of the safetensors container.

Layout: an 8-byte little-endian header length, a JSON header mapping each
tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets
relative to the end of the header), then the raw little-endian data.

The reference memory-maps each shard once and indexes name -> (dtype, shape,
bytes) (crates/synaptix-io/src/weights/safetensors.rs:85-109,233-255; dtype
table :13-24).  This reader does the same with ``mmap`` and hands out torch
tensors that alias the mapping; it checks what the container promises (header
inside the file, offsets inside the data, byte counts matching shape x dtype,
no name twice) and reports a violation with the tensor's name.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, List, Mapping, NamedTuple, Optional, Tuple

import torch


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


_DTYPES = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_DTYPE_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class TensorInfo(NamedTuple):
    dtype: str            # the container's dtype string, e.g. "BF16"
    shape: Tuple[int, ...]
    begin: int            # byte offsets inside the data section
    end: int


def _no_duplicate_keys(pairs):
    d = {}
    for k, v in pairs:
        if k in d:
            raise SafetensorsError(f"tensor name {k!r} appears twice in the header")
        d[k] = v
    return d


class SafetensorsFile:
    """One memory-mapped safetensors file."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open {path}: {e}") from e
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: truncated (no header length)")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: truncated (header of {hlen} bytes does not fit in {size})")
        raw = self._f.read(hlen)
        try:
            header = json.loads(raw.decode("utf-8"), object_pairs_hook=_no_duplicate_keys)
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", None) or {}
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self.tensors: Dict[str, TensorInfo] = {}
        for name, ent in header.items():
            try:
                dt = ent["dtype"]
                shape = tuple(int(s) for s in ent["shape"])
                b, e = (int(x) for x in ent["data_offsets"])
            except (KeyError, TypeError, ValueError) as ex:
                raise SafetensorsError(f"{path}: malformed entry for tensor {name!r}: {ex}") from ex
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r}")
            n = 1
            for s in shape:
                if s < 0:
                    raise SafetensorsError(f"{path}: tensor {name!r} has a negative dimension")
                n *= s
            want = n * _DTYPES[dt][1]
            if not (0 <= b <= e <= data_len):
                raise SafetensorsError(
                    f"{path}: truncated: tensor {name!r} spans bytes [{b}, {e}) but the data section holds {data_len}")
            if e - b != want:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} of shape {list(shape)} and dtype {dt} needs {want} bytes, header gives {e - b}")
            self.tensors[name] = TensorInfo(dt, shape, b, e)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self.tensors)

    def get(self, name: str) -> torch.Tensor:
        """The tensor as stored (a read-only view of the mapping; copy before writing to it)."""
        info = self.tensors[name]
        dtype, _ = _DTYPES[info.dtype]
        n = 1
        for s in info.shape:
            n *= s
        if n == 0:
            return torch.empty(info.shape, dtype=dtype)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the mapping is read-only; tensors are never written
            t = torch.frombuffer(self._mm, dtype=dtype, count=n, offset=self._data_start + info.begin)
        return t.reshape(info.shape)

    def close(self) -> None:
        # tensors handed out alias the mapping; leave closing to the garbage collector
        pass


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write ``tensors`` (CPU, any supported dtype) to ``path``; names are stored sorted."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _DTYPE_NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _DTYPE_NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((8 - len(raw) % 8) % 8)  # keep the data section 8-byte aligned
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                        t.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)


def resolve_shards(model_dir: str) -> List[str]:
    """``model.safetensors`` if present, else the sorted unique shard list of
    ``model.safetensors.index.json`` (crates/synaptix-models/llm/qwen3/src/loader.rs:87-115)."""
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        try:
            with open(index, "r", encoding="utf-8") as f:
                wm = json.load(f)["weight_map"]
        except (OSError, KeyError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{index}: cannot read weight_map: {e}") from e
        return [os.path.join(model_dir, s) for s in sorted(set(wm.values()))]
    raise SafetensorsError(
        f"{model_dir}: holds neither model.safetensors nor model.safetensors.index.json")
