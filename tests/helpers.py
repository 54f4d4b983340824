"""Shared pieces of the GPU tests: tolerances (fixed here, once), folders, oracles."""
import functools
import os
import tempfile

import torch

import plain_qwen3 as P
from tiny import CONFIGS, make_folder

# float32 engine against the float32 oracle: only summation order differs
F32_REL = 1e-4
# bfloat16 engine (bfloat16 weights, activations and cache; 32-bit sums) against the float32 oracle
BF16_REL = 3e-2
BF16_COS = 0.999

_FOLDERS = {}


def folder(name: str) -> str:
    if name not in _FOLDERS:
        _FOLDERS[name] = make_folder(name, tempfile.mkdtemp(prefix=f"sx_tiny_{name}_"))
    return _FOLDERS[name]


@functools.lru_cache(maxsize=None)
def oracle(name: str):
    return P.load_folder(folder(name))


@functools.lru_cache(maxsize=256)
def oracle_logits(name: str, tokens: tuple) -> torch.Tensor:
    cfg, W = oracle(name)
    return P.forward(cfg, W, list(tokens))


def assert_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = "") -> None:
    """``got`` and ``ref`` are [rows, vocab]; the scale is the oracle's largest logit."""
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = ref.abs().max().item()
    err = (got - ref).abs()
    rel = (err.max() / scale).item()
    if dtype == "float32":
        assert rel <= F32_REL, f"{what}: max|d|/max|logit| = {rel:.3e} > {F32_REL} at row {int(err.max(dim=1).values.argmax())}"
    else:
        assert rel <= BF16_REL, f"{what}: max|d|/max|logit| = {rel:.3e} > {BF16_REL} at row {int(err.max(dim=1).values.argmax())}"
        cos = torch.nn.functional.cosine_similarity(got, ref, dim=-1).min().item()
        assert cos >= BF16_COS, f"{what}: cosine {cos:.5f} < {BF16_COS}"


def poison_cache(engine) -> None:
    """Fill every cache page with NaN: a kernel that reads a place no step wrote shows at once."""
    for t in engine.cache._k + engine.cache._v:
        t.fill_(float("nan"))
