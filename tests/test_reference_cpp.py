"""The kernels' plain C++ counterparts (``synaptix_b200/csrc/reference.cpp``) against the plain Python
implementation of this folder, on the CPU: each operation alone, and a whole tiny model put together from
the C++ operations over a paged cache (whole prompts, and the last tokens one by one).  The GPU tests
compare every CUDA kernel with the same C++ functions (``tests/test_gpu_kernels_cpp.py``)."""
import math
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as P
import tiny
from synaptix_b200 import reference as R


def test_nothing_in_the_package_calls_the_cpu_reference():
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "synaptix_b200")
    for d, _, files in os.walk(root):
        for fn in files:
            if fn.endswith(".py") and fn != "reference.py":
                text = open(os.path.join(d, fn)).read()
                assert "reference import" not in text and "import reference" not in text and "load_host_library" not in text \
                    or fn == "build.py", f"{fn} uses the CPU reference"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_norm_and_residual(dtype):
    g = torch.Generator().manual_seed(1)
    E = torch.randn(50, 36, generator=g).to(dtype)
    ids = torch.tensor([3, 49, 0, 77, -1])
    out = R.embed_gather(E, ids)
    assert torch.equal(out[:3], E[ids[:3]].float()) and (out[3:] == 0).all()
    h = torch.randn(6, 36, generator=g) * 3
    delta = torch.randn(6, 36, generator=g).to(dtype)
    gain = 1 + 0.2 * torch.randn(36, generator=g)
    want_h = h + delta.float()
    h1 = h.clone()
    y = R.add_rmsnorm(h1, delta, gain, 2e-5, dtype)
    assert torch.equal(h1, want_h)
    tol = dict(atol=1e-6, rtol=1e-6) if dtype == torch.float32 else dict(atol=2e-2, rtol=1e-2)
    assert torch.allclose(y.float(), P.rms_norm(want_h, gain, 2e-5), **tol)
    h2 = h.clone()
    y2 = R.add_rmsnorm(h2, delta, gain, 2e-5, dtype, rows=torch.tensor([4, 1]), write_h=False)
    assert torch.equal(h2, h) and torch.equal(y2, y[[4, 1]])
    y3 = R.add_rmsnorm(h.clone(), None, gain, 2e-5, dtype)
    assert torch.allclose(y3.float(), P.rms_norm(h, gain, 2e-5), **tol)
    h4 = h.clone()
    R.residual_add(h4, delta)
    assert torch.equal(h4, want_h)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_products_and_silu_mul(dtype):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(7, 40, generator=g).to(dtype)
    w = (torch.randn(26, 40, generator=g) / 6).to(dtype)
    y = R.gemm(x, w, torch.float32)
    assert torch.allclose(y.double(), x.double() @ w.double().T, atol=1e-6, rtol=1e-6)
    assert R.gemm(x, w).dtype == dtype
    z = R.silu_mul(y.to(dtype))
    yy = y.to(dtype).float()
    want = yy[:, :13] / (1 + torch.exp(-yy[:, :13])) * yy[:, 13:]
    assert torch.allclose(z.float(), want, atol=1e-6 if dtype == torch.float32 else 2e-2, rtol=1e-2)
    # the feed-forward of the plain implementation from these two
    wd = (torch.randn(40, 13, generator=g) / 4).float()
    if dtype == torch.float32:
        ffn = R.gemm(R.silu_mul(R.gemm(x, w)), wd)
        assert torch.allclose(ffn, P.swiglu(x, w[:13], w[13:], wd), atol=1e-5, rtol=1e-5)


def _paged(keys, values, nkv, hd, dtype, seed):
    """Sequences' keys and values ``[n, nkv, hd]`` laid into pages in scrambled order; unused rows NaN."""
    g = torch.Generator().manual_seed(seed)
    need = [(k.shape[0] + 63) // 64 for k in keys]
    n_pages = sum(need) + 2
    perm = torch.randperm(n_pages - 1, generator=g).add(1).tolist()
    kp = torch.full((n_pages, nkv, 64, hd), float("nan"), dtype=dtype)
    vp = torch.full((n_pages, nkv, 64, hd), float("nan"), dtype=dtype)
    bt = torch.zeros((len(keys), max(need)), dtype=torch.int32)
    for s, (k, v) in enumerate(zip(keys, values)):
        for i in range(need[s]):
            page = perm.pop()
            bt[s, i] = page
            rows = min(64, k.shape[0] - 64 * i)
            kp[page, :, :rows] = k[64 * i:64 * i + rows].transpose(0, 1).to(dtype)
            vp[page, :, :rows] = v[64 * i:64 * i + rows].transpose(0, 1).to(dtype)
    return kp, vp, bt


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, None), (6, 2, 32, 50), (3, 3, 48, None), (8, 1, 80, 7)])
def test_attention_over_pages_matches_the_plain_attention(nh, nkv, hd, window):
    g = torch.Generator().manual_seed(nh * 100 + hd)
    lens = [70, 5, 131]
    qs = [torch.randn(n, nh, hd, generator=g) for n in lens]
    ks = [torch.randn(n, nkv, hd, generator=g) for n in lens]
    vs = [torch.randn(n, nkv, hd, generator=g) for n in lens]
    kp, vp, bt = _paged(ks, vs, nkv, hd, torch.float32, 5)
    q = torch.cat([x.reshape(-1, nh * hd) for x in qs])
    positions = torch.cat([torch.arange(n) for n in lens])
    seq_of = torch.cat([torch.full((n,), s) for s, n in enumerate(lens)])
    scale = 1 / math.sqrt(hd)
    out = R.attention(q, kp, vp, positions, seq_of, bt, nh, nkv, hd, scale, window)
    want = torch.cat([P.causal_gqa_attention(a, b, c, scale, window).reshape(-1, nh * hd) for a, b, c in zip(qs, ks, vs)])
    assert torch.isfinite(out).all() and torch.allclose(out, want, atol=2e-6, rtol=1e-5)
    # the last token of a sequence alone: the same row
    one = R.attention(qs[2][-1].reshape(1, -1), kp, vp, torch.tensor([130]), torch.tensor([2]), bt, nh, nkv, hd, scale, window)
    assert torch.allclose(one[0], want[-1], atol=2e-6, rtol=1e-5)


@pytest.mark.parametrize("nh,nkv,hd,rot", [(4, 2, 16, 16), (6, 2, 32, 32), (2, 1, 48, 32), (3, 3, 20, 0)])
def test_head_preparation_matches_the_plain_norm_and_rotation(nh, nkv, hd, rot):
    g = torch.Generator().manual_seed(hd)
    lens_past, lens_new = [3, 64], [5, 2]
    T = sum(lens_new)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g)
    wq, wk = 1 + 0.3 * torch.randn(hd, generator=g), 1 + 0.3 * torch.randn(hd, generator=g)
    inv = P.rotary_freqs(12345.0, rot) if rot else None
    positions = torch.cat([torch.arange(p, p + n) for p, n in zip(lens_past, lens_new)])
    seq_of = torch.cat([torch.full((n,), s) for s, n in enumerate(lens_new)])
    bt = torch.tensor([[2, 0], [3, 1]], dtype=torch.int32)
    kp = torch.full((4, nkv, 64, hd), float("nan"))
    vp = torch.full((4, nkv, 64, hd), float("nan"))
    eps = 3e-6
    q = R.qkv_prepare(qkv, kp, vp, wq, wk, inv, rot, eps, positions, seq_of, bt, nh, nkv, hd)
    x = qkv.view(T, nh + 2 * nkv, hd)
    qn, kn = P.rms_norm(x[:, :nh], wq, eps), P.rms_norm(x[:, nh:nh + nkv], wk, eps)
    if rot:
        qn = torch.cat([P.rope_rotate_half(qn[..., :rot], positions, inv), qn[..., rot:]], -1)
        kn = torch.cat([P.rope_rotate_half(kn[..., :rot], positions, inv), kn[..., rot:]], -1)
    assert torch.allclose(q.view(T, nh, hd), qn, atol=2e-6, rtol=1e-5)
    for t in range(T):
        page, row = bt[seq_of[t], positions[t] // 64], positions[t] % 64
        assert torch.allclose(kp[page, :, row], kn[t], atol=2e-6, rtol=1e-5)
        assert torch.equal(vp[page, :, row], x[t, nh + nkv:])
    assert torch.isnan(kp).sum() == kp.numel() - T * nkv * hd          # nothing else was written
    # a layer that reads another layer's cache writes nothing
    q2 = R.qkv_prepare(qkv, None, None, wq, wk, inv, rot, eps, positions, seq_of, bt, nh, nkv, hd)
    assert torch.equal(q2, q)


def test_argmax_penalties_and_sampling_match_the_plain_processors():
    x = torch.randn(5, 301)
    x[1, 5] = x[1, 299] = 40.0
    x[2, :] = 1.0
    assert R.argmax_rows(x).tolist() == [P.greedy(r) for r in x]
    x[3, 7] = float("nan")                                      # a NaN never wins
    assert R.argmax_rows(x)[3].item() == P.greedy(torch.nan_to_num(x[3], nan=-1e30))
    ctxs = [[1, 2, 2, 2, 7, 300], [3] * 10 + [4], [5, 6, 7, 8, 9, 5, 5]]
    y0 = torch.randn(3, 301) * 3
    for last_n in (0, 4):
        hist = torch.zeros(3, 11, dtype=torch.int32)
        for r, c in enumerate(ctxs):
            hist[r, :len(c)] = torch.tensor(c)
        y = y0.clone()
        R.apply_penalties(y, hist, torch.tensor([len(c) for c in ctxs]), last_n, 1.3, 0.5, 0.25)
        for r in range(3):
            ref = P.processed_logits(y0[r].numpy(), ctxs[r], repetition_penalty=1.3, repeat_last_n=last_n, presence_penalty=0.5,
                                     frequency_penalty=0.25)
            assert np.allclose(y[r].numpy(), ref, atol=1e-6)
    V, Rr, seed = 1001, 48, 4321
    z = torch.randn(Rr, V) * 2.5
    z[0, 17] = z[1, 0] = float("nan")                           # a NaN is never kept and never the cut-off
    z[2, :500] = float("-inf")
    seq, step = torch.arange(Rr) % 5, torch.arange(Rr)
    for kw in (dict(temperature=1.0), dict(temperature=0.7, top_k=5), dict(temperature=1.2, top_p=0.6),
               dict(temperature=1.0, min_p=0.2), dict(temperature=0.9, top_k=40, top_p=0.8, min_p=0.05)):
        got, u, kept = R.sample_rows(z, kw["temperature"], kw.get("top_k", 0), kw.get("top_p", 1.0), kw.get("min_p", 0.0), seed,
                                     seq, step, want_kept=True)
        for r in range(Rr):
            u_ref = float(P.uniform_from_u32(P.philox_u32(seed, int(step[r]), int(seq[r]))))
            assert float(u[r]) == u_ref
            # what the reference does with a NaN depends on its sort; here a NaN counts as -inf everywhere
            v = P.processed_logits(np.nan_to_num(z[r].numpy(), nan=-np.inf, posinf=np.inf, neginf=-np.inf), **kw)
            assert np.array_equal(np.isfinite(v), kept[r].numpy().astype(bool)), f"{kw} row {r}: kept sets differ"
            cum = P.multinomial_intervals(v)
            t = int(got[r])
            lo = cum[t - 1] if t > 0 else 0.0
            assert lo - 1e-5 <= u_ref <= cum[t] + 1e-5
    got, _, _ = R.sample_rows(z, 0.0, 0, 1.0, 0.0, seed, seq, step)
    assert got.tolist() == torch.nan_to_num(z, nan=float("-inf")).argmax(1).tolist()


def test_decode_bookkeeping():
    tok = torch.tensor([5, 6, 7], dtype=torch.int32)
    hist = torch.zeros(3, 4, dtype=torch.int32)
    hl = torch.tensor([1, 2, 1], dtype=torch.int32)
    hist[:, 0] = torch.tensor([5, 9, 7])
    hist[1, 1] = 6
    R.decode_begin(tok, torch.tensor([-1, 11, -1], dtype=torch.int32), hist, hl)
    assert tok.tolist() == [5, 11, 7] and hist[1].tolist() == [9, 11, 0, 0]
    pos, past, lens, rs = (torch.tensor(v, dtype=torch.int32) for v in ([4, 9, 0], [4, 9, 0], [5, 10, 1], [0, 3, 0]))
    R.decode_advance(tok, torch.tensor([21, 22, 23], dtype=torch.int32), pos, past, lens, rs,
                     torch.tensor([1, 1, 0], dtype=torch.int32), hist, hl)
    assert tok.tolist() == [21, 22, 7] and pos.tolist() == [5, 10, 0] and lens.tolist() == [6, 11, 1]
    assert rs.tolist() == [1, 4, 0] and hl.tolist() == [2, 3, 1] and hist[0].tolist() == [5, 21, 0, 0]


# ----------------------------------------------------------------------------------------
# a whole model from the C++ operations, over a paged cache
# ----------------------------------------------------------------------------------------
class CppModel:
    """The decoder stepped with the C++ operations only: one packed step of any tokens of any sequences."""

    def __init__(self, cfg, W, n_pages=12, max_pages=4):
        self.cfg, self.W = cfg, W
        self.nh, self.nkv, self.hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], P.head_dim_of(cfg)
        L = cfg["num_hidden_layers"]
        self.k = [torch.full((n_pages, self.nkv, 64, self.hd), float("nan")) for _ in range(L)]
        self.v = [torch.full((n_pages, self.nkv, 64, self.hd), float("nan")) for _ in range(L)]
        self.inv = P.rotary_freqs(P.rope_theta_of(cfg), self.hd)
        self.free = list(range(n_pages - 1, 0, -1))
        self.bt = {}                                        # sequence -> list of pages
        self.len = {}
        self.max_pages = max_pages

    def step(self, entries):
        """entries: [(sequence id, tokens)]; returns the logits of every token, packed."""
        cfg, W = self.cfg, self.W
        ids, positions, seq_of = [], [], []
        order = sorted({s for s, _ in entries} | set(self.bt))
        for s, toks in entries:
            past = self.len.get(s, 0)
            pages = self.bt.setdefault(s, [])
            while len(pages) * 64 < past + len(toks):
                pages.append(self.free.pop())
            ids += list(toks)
            positions += list(range(past, past + len(toks)))
            seq_of += [order.index(s)] * len(toks)
            self.len[s] = past + len(toks)
        bt = torch.zeros((len(order), self.max_pages), dtype=torch.int32)
        for i, s in enumerate(order):
            bt[i, :len(self.bt.get(s, []))] = torch.tensor(self.bt.get(s, []), dtype=torch.int32)
        positions, seq_of = torch.tensor(positions), torch.tensor(seq_of)
        eps = cfg["rms_norm_eps"]
        h = R.embed_gather(W["model.embed_tokens.weight"], torch.tensor(ids))
        delta = None
        for layer in range(cfg["num_hidden_layers"]):
            p = f"model.layers.{layer}."
            x = R.add_rmsnorm(h, delta, W[p + "input_layernorm.weight"], eps, torch.float32)
            wqkv = torch.cat([W[p + f"self_attn.{n}_proj.weight"] for n in "qkv"])
            q = R.qkv_prepare(R.gemm(x, wqkv), self.k[layer], self.v[layer], W[p + "self_attn.q_norm.weight"],
                              W[p + "self_attn.k_norm.weight"], self.inv, self.hd, eps, positions, seq_of, bt, self.nh, self.nkv,
                              self.hd)
            a = R.attention(q, self.k[layer], self.v[layer], positions, seq_of, bt, self.nh, self.nkv, self.hd,
                            1 / math.sqrt(self.hd), P.layer_window(cfg, layer))
            x = R.add_rmsnorm(h, R.gemm(a, W[p + "self_attn.o_proj.weight"]), W[p + "post_attention_layernorm.weight"], eps,
                              torch.float32)
            wgu = torch.cat([W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"]])
            delta = R.gemm(R.silu_mul(R.gemm(x, wgu)), W[p + "mlp.down_proj.weight"])
        x = R.add_rmsnorm(h, delta, W["model.norm.weight"], eps, torch.float32)
        tied = cfg.get("tie_word_embeddings")
        head = W["model.embed_tokens.weight"] if (tied or "lm_head.weight" not in W) else W["lm_head.weight"]
        return R.gemm(x, head)


@pytest.mark.parametrize("name", ["A", "B", "W"])
def test_a_whole_model_from_the_cpp_operations(tmp_path, name):
    cfg, W = P.load_folder(tiny.make_folder(name, str(tmp_path)))
    W = {k: v.float() for k, v in W.items()}
    prompts = [tiny.random_tokens(cfg["vocab_size"], n, 7 + n) for n in (70, 9, 33)]
    want = [P.forward(cfg, W, p) for p in prompts]
    scale = max(w.abs().max().item() for w in want)
    m = CppModel(cfg, W)
    # all prompts whole, in one packed step
    lg = m.step(list(enumerate(prompts)))
    at = 0
    for p, w in zip(prompts, want):
        assert (lg[at:at + len(p)] - w).abs().max().item() <= 1e-4 * scale
        at += len(p)
    # the same with the last five tokens of each one by one, the shorter ones first in the batch
    m = CppModel(cfg, W)
    m.step([(i, p[:-5]) for i, p in enumerate(prompts)])
    for j in range(5, 0, -1):
        lg = m.step([(i, [p[len(p) - j]]) for i, p in reversed(list(enumerate(prompts)))])
        for row, (i, p) in enumerate(reversed(list(enumerate(prompts)))):
            assert (lg[row] - want[i][len(p) - j]).abs().max().item() <= 1e-4 * scale
