"""The plain implementation against outputs of the reference's OWN op-level oracles.

tests/golden/reference_ops.safetensors holds sliced OUTPUTS of the reference's PyTorch generator
functions (scripts/reference/gen_*.py), made by tests/golden/make_golden.py.  The inputs are
not stored: each test below regenerates them with the seed, shapes and order of draws that the
generator function uses (cited beside each), which torch's CPU generator reproduces exactly.
The reference's Rust tests hold its kernels to these tensors at 1e-5
(crates/synaptix-test-utils/src/lib.rs:43-90); the same bound is used here.
"""
import math
import os

import numpy as np
import torch

import plain_qwen3 as P
from safetensors import safe_open          # the package's reader: this anchor shares no code with the product

TOL = 1e-5
_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_ops.safetensors")


def _golden():
    with safe_open(_PATH, framework="pt") as f:
        return {name: f.get_tensor(name).clone() for name in f.keys()}


def _close(got, want):
    assert got.shape == want.shape
    assert torch.allclose(got, want, rtol=TOL, atol=TOL), float((got - want).abs().max())


def test_rms_norm():
    # scripts/reference/gen_norm.py:27-35: seed 0, x [4,32,256], weight = 1 + randn(256)*0.02, eps 1e-6
    g = _golden()
    torch.manual_seed(0)
    x = torch.randn(4, 32, 256, dtype=torch.float32)
    w = torch.ones(256, dtype=torch.float32) + torch.randn(256) * 0.02
    _close(P.rms_norm(x[0, :4], w, 1e-6), g["rms_norm.output"])


def test_rotate_half():
    # scripts/reference/gen_pos.py:43-60: seed 0, q then k [2,8,32,64], base 10000, positions 0..31
    g = _golden()
    torch.manual_seed(0)
    q = torch.randn(2, 8, 32, 64, dtype=torch.float32)
    k = torch.randn(2, 8, 32, 64, dtype=torch.float32)
    freqs = P.rotary_freqs(10000.0, 64)
    pos = torch.arange(32)
    for src, key in ((q, "rope_split.q_out"), (k, "rope_split.k_out")):
        x = src[0, :2].permute(1, 0, 2)                                   # [T, heads, d]
        _close(P.rope_rotate_half(x, pos, freqs).permute(1, 0, 2), g[key])


def test_swiglu():
    # scripts/reference/gen_ffn.py:44-57: seed 1, x [2,16,256], w1 (gate) [512,256], w2 (down)
    # [256,512], w3 (up) [512,256], each randn*0.02, drawn in that order
    g = _golden()
    torch.manual_seed(1)
    x = torch.randn(2, 16, 256, dtype=torch.float32)
    w1 = torch.randn(512, 256, dtype=torch.float32) * 0.02
    w2 = torch.randn(256, 512, dtype=torch.float32) * 0.02
    w3 = torch.randn(512, 256, dtype=torch.float32) * 0.02
    _close(P.swiglu(x[0, :4], w1, w3, w2), g["swiglu.output"])


def test_causal_attention():
    # scripts/reference/gen_attention.py:36-43: seed 1, q, k, v [2,8,32,64], causal, scale 1/sqrt(64)
    g = _golden()
    torch.manual_seed(1)
    q, k, v = (torch.randn(2, 8, 32, 64, dtype=torch.float32) for _ in range(3))
    to_t = lambda a: a[0, :2].permute(1, 0, 2).contiguous()
    out = P.causal_gqa_attention(to_t(q), to_t(k), to_t(v), 1.0 / math.sqrt(64))
    _close(out.permute(1, 0, 2), g["sdpa_causal.output"])


def test_grouped_heads():
    # scripts/reference/gen_attention.py:46-56: seed 2, q [2,8,32,64], k and v [2,2,32,64];
    # query head h reads kv head h // 4 (repeat_interleave)
    g = _golden()
    torch.manual_seed(2)
    q = torch.randn(2, 8, 32, 64, dtype=torch.float32)
    k = torch.randn(2, 2, 32, 64, dtype=torch.float32)
    v = torch.randn(2, 2, 32, 64, dtype=torch.float32)
    to_t = lambda a: a[1].permute(1, 0, 2).contiguous()
    out = P.causal_gqa_attention(to_t(q), to_t(k), to_t(v), 1.0 / math.sqrt(64)).permute(1, 0, 2)
    _close(out[[0, 3, 4, 7]], g["gqa.output"])


def test_greedy():
    # scripts/reference/gen_infer.py:29-33: seed 0, logits [4,32000]
    g = _golden()
    torch.manual_seed(0)
    logits = torch.randn(4, 32000, dtype=torch.float32)
    assert [P.greedy(row) for row in logits] == g["greedy.tokens"].tolist()


def test_temperature():
    # scripts/reference/gen_infer.py:36-49: seed 1, logits [4,32000], temperature 0.8, softmax
    g = _golden()
    rows, vocab = int(g["temperature.vocab"][1]), int(g["temperature.vocab"][0])
    torch.manual_seed(1)
    logits = torch.randn(rows, vocab, dtype=torch.float32)
    for r in range(2):
        v = P.processed_logits(logits[r].numpy(), temperature=0.8)
        _close(torch.from_numpy(v[:64]), g["temperature.scaled_logits"][r])
        cum = P.multinomial_intervals(v)
        probs = np.diff(np.concatenate([[0.0], cum]))[:64]
        want = g["temperature.probs"][r].numpy()
        # probabilities are near 1/vocab, so the bound is relative: float32 softmax over 32000
        # entries against the float64 one here
        assert np.allclose(probs, want, rtol=1e-4, atol=1e-9), float(np.abs(probs - want).max())
