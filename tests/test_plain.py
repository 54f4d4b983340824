"""The plain implementation checked against itself and against first principles (CPU)."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from tiny import make_folder, random_tokens


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: P.load_folder(make_folder(n, str(tmp_path_factory.mktemp(n)))) for n in "ABW"}


def test_rms_norm_against_explicit_loops():
    x = torch.randn(3, 7)
    w = torch.randn(7)
    y = P.rms_norm(x, w, 1e-5)
    for r in range(3):
        ms = sum(float(v) ** 2 for v in x[r]) / 7
        for c in range(7):
            assert abs(float(y[r, c]) - float(x[r, c]) / math.sqrt(ms + 1e-5) * float(w[c])) < 1e-5


def test_rotation_keeps_norms_and_depends_on_distance_only():
    f = P.rotary_freqs(10000.0, 16)
    assert abs(float(f[0]) - 1.0) < 1e-7 and abs(float(f[4]) - 10000.0 ** (-8 / 16)) < 1e-7
    q = torch.randn(1, 1, 16)
    k = torch.randn(1, 1, 16)
    def dot(pq, pk):
        a = P.rope_rotate_half(q, torch.tensor([pq]), f)
        b = P.rope_rotate_half(k, torch.tensor([pk]), f)
        return float((a * b).sum())
    assert abs(float(P.rope_rotate_half(q, torch.tensor([37]), f).norm()) - float(q.norm())) < 1e-5
    assert abs(dot(5, 2) - dot(45, 42)) < 1e-4
    assert abs(dot(0, 0) - float((q * k).sum())) < 1e-6
    # rotate-half pairs element i with i + d/2
    x = torch.zeros(1, 1, 16); x[0, 0, 3] = 1.0
    y = P.rope_rotate_half(x, torch.tensor([1]), f)
    ang = float(f[3])
    assert abs(float(y[0, 0, 3]) - math.cos(ang)) < 1e-6 and abs(float(y[0, 0, 11]) - math.sin(ang)) < 1e-6


def test_attention_against_explicit_loops():
    T, nh, nkv, d = 6, 4, 2, 8
    q, k, v = torch.randn(T, nh, d), torch.randn(T, nkv, d), torch.randn(T, nkv, d)
    for window in (None, 3):
        o = P.causal_gqa_attention(q, k, v, 0.3, window)
        for i in range(T):
            for h in range(nh):
                kh = h // 2
                js = [j for j in range(T) if j <= i and (window is None or j > i - window)]
                s = [float(q[i, h] @ k[j, kh]) * 0.3 for j in js]
                m = max(s)
                e = [math.exp(x - m) for x in s]
                z = sum(e)
                ref = sum((e[a] / z) * v[js[a], kh] for a in range(len(js)))
                assert torch.allclose(o[i, h], ref, atol=1e-5)


def test_window_at_least_sequence_is_full_attention():
    T = 9
    q, k, v = torch.randn(T, 2, 4), torch.randn(T, 1, 4), torch.randn(T, 1, 4)
    assert torch.allclose(P.causal_gqa_attention(q, k, v, 0.5, None), P.causal_gqa_attention(q, k, v, 0.5, T))
    assert not torch.allclose(P.causal_gqa_attention(q, k, v, 0.5, None), P.causal_gqa_attention(q, k, v, 0.5, 2))


def test_swiglu_against_explicit():
    x, wg, wu, wd = torch.randn(2, 5), torch.randn(7, 5), torch.randn(7, 5), torch.randn(5, 7)
    g, u = x @ wg.T, x @ wu.T
    ref = (g * torch.sigmoid(g) * u) @ wd.T
    assert torch.allclose(P.swiglu(x, wg, wu, wd), ref, atol=1e-5)


def test_logits_do_not_depend_on_later_tokens(folders):
    for name, (cfg, W) in folders.items():
        a = random_tokens(cfg["vocab_size"], 40, 1)
        b = a[:25] + random_tokens(cfg["vocab_size"], 15, 2)
        la, lb = P.forward(cfg, W, a), P.forward(cfg, W, b)
        assert torch.allclose(la[:25], lb[:25], atol=1e-5), name
        assert not torch.allclose(la[25:], lb[25:], atol=1e-5)


def test_window_config_changes_late_positions_only(folders):
    cfg, W = folders["W"]
    full = dict(cfg, use_sliding_window=False)
    t = random_tokens(cfg["vocab_size"], 60, 3)
    lw, lf = P.forward(cfg, W, t), P.forward(full, W, t)
    assert torch.allclose(lw[:24], lf[:24], atol=1e-5)       # up to the window nothing is cut
    assert not torch.allclose(lw[30:], lf[30:], atol=1e-4)


def test_tied_and_untied_heads(folders):
    cfg, W = folders["A"]
    assert "lm_head.weight" not in W
    cfgb, Wb = folders["B"]
    assert Wb["lm_head.weight"].shape == (389, 96)
    assert Wb["model.norm.weight"].dtype == torch.float32


def test_philox_known_answer():
    # crates/synaptix-ops/src/rng.rs:163-168
    assert P.philox4x32((0, 0, 0, 0), (0, 0)) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert P.philox_u32(0, 0) == 0x6627E8D5 and P.philox_u32(0, 3) == 0x9B00DBD8
    assert P.philox_u32(0, 4) == P.philox4x32((1, 0, 0, 0), (0, 0))[0]


def test_processors_follow_the_reference_unit_tests():
    # crates/synaptix-infer/src/sampling/repetition.rs:79-133
    v = np.array([1.0, 1.0, 1.0, 1.0], dtype=np.float32)
    P.apply_repetition(v, [0, 1, 2, 3], 2.0, 2)
    assert list(v) == [1.0, 1.0, 0.5, 0.5]
    v = np.array([-1.0], dtype=np.float32)
    P.apply_repetition(v, [0], 2.0, 0)
    assert v[0] == -2.0
    v = np.zeros(2, dtype=np.float32)
    P.apply_presence_frequency(v, [0, 0, 0, 1], 0.5, 0.25, 0)
    assert abs(v[0] + 1.25) < 1e-6 and abs(v[1] + 0.75) < 1e-6
    v = np.array([1.0, 3.0, 2.0, 0.0], dtype=np.float32)
    P.filter_top_k(v, 2)
    assert list(np.isfinite(v)) == [False, True, True, False]
    v = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32))
    P.filter_top_p(v, 0.7)          # sums before each: 0, .5, .8 -> the third is cut
    assert list(np.isfinite(v)) == [True, True, False, False]
    v = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32))
    P.filter_min_p(v, 0.5)
    assert list(np.isfinite(v)) == [True, True, False, False]
    assert P.greedy(torch.tensor([0.0, 2.0, 2.0, 1.0])) == 2          # the last of equal maxima
    assert P.multinomial(np.log(np.array([0.25, 0.25, 0.5], dtype=np.float32)), 0.6) == 2
