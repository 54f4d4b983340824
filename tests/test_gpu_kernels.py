"""Each kernel alone against a plain float32 reference of the same operation, at sizes other
than the engine tests use.  Inputs are made so that faults show: pages in scrambled order,
unused cache filled with NaN, one far key whose score stands out, keys at a window's edge."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu

DT = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def dev(t, dtype=None):
    t = t.to("cuda")
    return t.to(dtype) if dtype is not None else t


def make_paged(seqs_k, seqs_v, nkv, hd, dtype, seed=0):
    """Dense per-sequence K/V [len, nkv, hd] -> NaN-filled pages in scrambled order + block table."""
    g = torch.Generator().manual_seed(seed)
    need = [(k.shape[0] + 63) // 64 for k in seqs_k]
    n_pages = sum(need) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    kp = torch.full((n_pages, nkv, 64, hd), float("nan"), dtype=dtype)
    vp = torch.full((n_pages, nkv, 64, hd), float("nan"), dtype=dtype)
    maxp = max(need)
    bt = torch.zeros((len(seqs_k), maxp), dtype=torch.int32)
    for s, (k, v) in enumerate(zip(seqs_k, seqs_v)):
        for i in range(need[s]):
            page = perm.pop()
            bt[s, i] = page
            n = min(64, k.shape[0] - 64 * i)
            kp[page, :, :n] = k[64 * i:64 * i + n].transpose(0, 1).to(dtype)
            vp[page, :, :n] = v[64 * i:64 * i + n].transpose(0, 1).to(dtype)
    return kp.cuda(), vp.cuda(), bt.cuda()


@pytest.mark.parametrize("dtype", DT)
def test_embed_gather(dtype):
    from synaptix_b200 import ops
    table = torch.randn(1000, 200).to(dtype)
    ids = torch.tensor([0, 999, 5, 5, 123], dtype=torch.int32)
    out = ops.embed_gather(dev(table), dev(ids))
    assert out.dtype == torch.float32
    assert torch.equal(out.cpu(), table.float()[ids.long()])


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("H", [7, 300, 2560])
def test_add_rmsnorm(dtype, H):
    from synaptix_b200 import ops
    T = 9
    h = torch.randn(T, H) * 3
    d = torch.randn(T, H).to(dtype)
    w = 1 + 0.2 * torch.randn(H)
    eps = 1e-5
    hd = dev(h.clone())
    y = ops.add_rmsnorm(hd, dev(d), dev(w), eps, dtype)
    s = h + d.float()
    assert torch.allclose(hd.cpu(), s, atol=1e-6)                       # the sum is kept in 32-bit
    assert torch.allclose(y.float().cpu(), P.rms_norm(s, w, eps), **tol(dtype))
    # without delta; and gathered rows leave h alone
    hd = dev(h.clone())
    y = ops.add_rmsnorm(hd, None, dev(w), eps, dtype)
    assert torch.allclose(y.float().cpu(), P.rms_norm(h, w, eps), **tol(dtype))
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    y = ops.add_rmsnorm(hd, dev(d), dev(w), eps, dtype, rows=dev(rows))
    assert torch.equal(hd.cpu(), h)
    assert torch.allclose(y.float().cpu(), P.rms_norm(s[rows.long()], w, eps), **tol(dtype))


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("M,N,K", [(1, 389, 77), (5, 64, 96), (16, 130, 33), (17, 200, 160), (100, 389, 250), (130, 70, 1)])
def test_gemm_generic(dtype, M, N, K):
    from synaptix_b200 import ops
    a = torch.randn(M, K).to(dtype)
    w = torch.randn(N, K).to(dtype)
    ref = a.double() @ w.double().T
    out = ops.gemm_generic(dev(a), dev(w), out_dtype=torch.float32)
    assert torch.allclose(out.cpu().double(), ref, atol=1e-4 * math.sqrt(K), rtol=1e-5)
    out = ops.gemm_generic(dev(a), dev(w))
    assert out.dtype == dtype
    assert torch.allclose(out.float().cpu().double(), ref, atol=(1e-4 if dtype == torch.float32 else 0.08) * math.sqrt(K), rtol=tol(dtype)["rtol"])


@pytest.mark.parametrize("dtype", DT)
def test_silu_mul(dtype):
    from synaptix_b200 import ops
    gu = (torch.randn(5, 2 * 37) * 4).to(dtype)
    g, u = gu.float()[:, :37], gu.float()[:, 37:]
    out = ops.silu_mul(dev(gu))
    assert torch.allclose(out.float().cpu(), g / (1 + torch.exp(-g)) * u, **tol(dtype))


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd,rot,norm", [(4, 2, 16, 16, True), (6, 2, 32, 32, True), (5, 1, 48, 24, True),
                                                 (3, 3, 80, 80, False), (2, 1, 256, 0, True),
                                                 # head sizes 64 and 128 (the wide bfloat16 kernel): head counts that do
                                                 # not fill a warp's group, no rotation, no norm, the benchmark's counts
                                                 (5, 1, 128, 128, True), (6, 3, 64, 64, True), (3, 1, 128, 0, False),
                                                 (7, 7, 64, 0, True), (32, 8, 128, 128, True)])
def test_qkv_prepare_norm_rotation_and_cache_write(dtype, nh, nkv, hd, rot, norm):
    from synaptix_b200 import ops
    from synaptix_b200.parts import rotary_inv_freq
    lens_past, lens_new = [0, 70, 63], [5, 1, 66]
    eps, theta = 1e-5, 5000.0
    S = len(lens_new)
    T = sum(lens_new)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd).to(dtype)
    wq, wk = 1 + 0.3 * torch.randn(hd), 1 + 0.3 * torch.randn(hd)
    pos = torch.cat([torch.arange(p, p + n) for p, n in zip(lens_past, lens_new)]).to(torch.int32)
    sot = torch.cat([torch.full((n,), i) for i, n in enumerate(lens_new)]).to(torch.int32)
    # pages: empty sequences of the final lengths, NaN everywhere
    zeros = [torch.zeros(p + n, nkv, hd) for p, n in zip(lens_past, lens_new)]
    kp, vp, bt = make_paged(zeros, zeros, nkv, hd, dtype, seed=1)
    kp.fill_(float("nan")); vp.fill_(float("nan"))
    q_out = torch.empty(T, nh * hd, dtype=dtype, device="cuda")
    inv = torch.from_numpy(rotary_inv_freq(theta, rot)).cuda() if rot else None
    ops.qkv_prepare(dev(qkv), q_out, kp, vp, dev(wq) if norm else None, dev(wk) if norm else None, inv, rot, eps,
                    dev(pos), dev(sot), bt, nh, nkv, hd)
    x = qkv.float()
    q = x[:, :nh * hd].view(T, nh, hd)
    k = x[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd)
    v = x[:, (nh + nkv) * hd:].view(T, nkv, hd)
    if norm:
        q, k = P.rms_norm(q, wq, eps), P.rms_norm(k, wk, eps)
    if rot:
        f = P.rotary_freqs(theta, rot)
        q = torch.cat([P.rope_rotate_half(q[..., :rot], pos, f), q[..., rot:]], -1)
        k = torch.cat([P.rope_rotate_half(k[..., :rot], pos, f), k[..., rot:]], -1)
    assert torch.allclose(q_out.float().cpu().view(T, nh, hd), q, **tol(dtype))
    kpc, vpc, btc = kp.float().cpu(), vp.float().cpu(), bt.cpu()
    written = torch.zeros(kpc.shape[0], 64, dtype=torch.bool)
    for t in range(T):
        s, p = int(sot[t]), int(pos[t])
        page = int(btc[s, p // 64])
        assert torch.allclose(kpc[page, :, p % 64], k[t], **tol(dtype))
        assert torch.allclose(vpc[page, :, p % 64], v[t], **tol(dtype))
        written[page, p % 64] = True
    # nothing else was touched
    assert torch.isnan(kpc.permute(0, 2, 1, 3)[~written]).all() and torch.isnan(vpc.permute(0, 2, 1, 3)[~written]).all()
    # a layer that reads another layer's cache writes nothing
    q2 = torch.empty_like(q_out)
    ops.qkv_prepare(dev(qkv), q2, None, None, dev(wq) if norm else None, dev(wk) if norm else None, inv, rot, eps,
                    dev(pos), dev(sot), bt, nh, nkv, hd)
    assert torch.equal(q2, q_out)


def attention_reference(q, ks, vs, positions, sot, scale, window):
    """q [T, nh, hd]; ks/vs dense per sequence; each token attends within its own sequence."""
    T, nh, hd = q.shape
    out = torch.empty(T, nh, hd, dtype=torch.float64)
    for t in range(T):
        s, p = int(sot[t]), int(positions[t])
        lo = 0 if window is None else max(0, p - window + 1)
        k, v = ks[s][lo:p + 1].double(), vs[s][lo:p + 1].double()
        g = nh // k.shape[1]
        for h in range(nh):
            sc = (k[:, h // g] @ q[t, h].double()) * scale
            pr = torch.softmax(sc, 0)
            out[t, h] = pr @ v[:, h // g]
    return out.float()


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, None), (6, 2, 32, None), (5, 1, 48, 24), (8, 8, 64, None),
                                               (8, 2, 128, 100), (2, 1, 256, None), (3, 1, 80, None)])
def test_attention_generic(dtype, nh, nkv, hd, window):
    from synaptix_b200 import ops
    past, new = [0, 130, 200, 64], [67, 1, 3, 1]
    ks = [torch.randn(p + n, nkv, hd).to(dtype).float() for p, n in zip(past, new)]
    vs = [torch.randn(p + n, nkv, hd).to(dtype).float() for p, n in zip(past, new)]
    kp, vp, bt = make_paged(ks, vs, nkv, hd, dtype, seed=2)
    T = sum(new)
    q = torch.randn(T, nh, hd).to(dtype)
    pos = torch.cat([torch.arange(p, p + n) for p, n in zip(past, new)]).to(torch.int32)
    sot = torch.cat([torch.full((n,), i) for i, n in enumerate(new)]).to(torch.int32)
    scale = 1 / math.sqrt(hd)
    out = ops.attn_generic(dev(q.view(T, nh * hd)), kp, vp, dev(pos), dev(sot), bt, nh, nkv, hd, scale, window)
    ref = attention_reference(q.float(), ks, vs, pos, sot, scale, window)
    assert torch.allclose(out.float().cpu().view(T, nh, hd), ref, **tol(dtype))


@pytest.mark.parametrize("dtype", DT)
def test_attention_finds_one_far_key_among_hundreds(dtype):
    """One key, far back, is scaled so that its score stands out: the output must be its value."""
    from synaptix_b200 import ops
    nh, nkv, hd, L = 4, 2, 64, 700
    for far in (0, 1, 63, 64, 333, 698, 699):
        k = torch.randn(L, nkv, hd) * 0.1
        v = torch.randn(L, nkv, hd)
        q = torch.randn(1, nh, hd)
        # make key `far` of each kv head parallel to the mean query of its group, and long
        for kh in range(nkv):
            k[far, kh] = q[0, kh * 2] / q[0, kh * 2].norm() * 40.0
        q[0, 1], q[0, 3] = q[0, 0].clone(), q[0, 2].clone()
        kp, vp, bt = make_paged([k], [v], nkv, hd, dtype, seed=far)
        pos = torch.tensor([L - 1], dtype=torch.int32)
        sot = torch.zeros(1, dtype=torch.int32)
        out = ops.attn_generic(dev(q.view(1, nh * hd), dtype), kp, vp, dev(pos), dev(sot), bt, nh, nkv, hd, 1.0, None)
        out = out.float().cpu().view(nh, hd)
        for h in range(nh):
            assert torch.allclose(out[h], v[far, h // 2].to(dtype).float(), atol=2e-2), f"far key {far}, head {h}"


@pytest.mark.parametrize("dtype", DT)
def test_attention_window_edge(dtype):
    """The key just outside the window has a huge score and a huge value: it must not count;
    the key just inside is the one that stands out."""
    from synaptix_b200 import ops
    nh, nkv, hd, W = 2, 1, 32, 70
    for p in (69, 70, 71, 133, 134, 200):
        L = p + 1
        k = torch.randn(L, nkv, hd) * 0.05
        v = torch.randn(L, nkv, hd)
        q = torch.randn(1, nh, hd)
        q[0, 1] = q[0, 0]
        unit = q[0, 0] / q[0, 0].norm()
        inside, outside = p - W + 1, p - W
        if inside >= 0:
            k[inside, 0] = unit * 30.0
        if outside >= 0:
            k[outside, 0] = unit * 60.0
            v[outside, 0] = 1000.0
        kp, vp, bt = make_paged([k], [v], nkv, hd, dtype, seed=p)
        out = ops.attn_generic(dev(q.view(1, nh * hd), dtype), kp, vp, dev(torch.tensor([p], dtype=torch.int32)),
                               dev(torch.zeros(1, dtype=torch.int32)), bt, nh, nkv, hd, 1.0, W)
        out = out.float().cpu().view(nh, hd)
        if inside >= 0:
            assert torch.allclose(out[0], v[inside, 0].to(dtype).float(), atol=2e-2), f"position {p}"
        assert out.abs().max() < 50, f"position {p}: a key outside the window was used"


def test_argmax_last_of_equal_maxima():
    from synaptix_b200.ops import sampling as K
    x = torch.randn(5, 3001)
    x[0, 17] = 50.0
    x[1, 5] = x[1, 2999] = 40.0
    x[2, :] = 1.0
    x[3, 3000] = 60.0
    x[4, 0] = 70.0
    got = K.argmax_rows(x.cuda()).tolist()
    assert got == [17, 2999, 3000, 3000, 0]
    assert got == [P.greedy(r) for r in x]


def test_argmax_wide_rows_in_chunks():
    from synaptix_b200.ops import sampling as K
    x = torch.randn(9, 151936)
    x[0, 151935] = 9.0
    x[1, 0] = 9.0
    x[2, 70000] = x[2, 4096] = x[2, 4095] = 9.0          # equal maxima in different chunks: the last one wins
    x[3, :] = 0.5
    got = K.argmax_rows(x.cuda()).tolist()
    assert got == [P.greedy(r) for r in x]
    assert got[:4] == [151935, 0, 70000, 151935]


def test_penalties_match_the_plain_processors():
    from synaptix_b200.ops import sampling as K
    V = 500
    x = torch.randn(3, V) * 3
    ctxs = [[1, 2, 2, 2, 7, 499], [3] * 10 + [4], [5, 6, 7, 8, 9, 5, 5]]
    for last_n in (0, 4):
        hist = torch.zeros(3, 11, dtype=torch.int32)
        lens = torch.tensor([len(c) for c in ctxs], dtype=torch.int32)
        for r, c in enumerate(ctxs):
            hist[r, :len(c)] = torch.tensor(c)
        y = x.clone().cuda()
        K.apply_penalties(y, hist.cuda(), lens.cuda(), last_n, 1.3, 0.5, 0.25)
        for r in range(3):
            ref = P.processed_logits(x[r].numpy(), ctxs[r], repetition_penalty=1.3, repeat_last_n=last_n,
                                     presence_penalty=0.5, frequency_penalty=0.25)
            assert np.allclose(y[r].cpu().numpy(), ref, atol=1e-5)


@pytest.mark.parametrize("kw", [dict(temperature=1.0), dict(temperature=0.7), dict(temperature=0.8, top_k=5),
                                dict(temperature=1.2, top_p=0.6), dict(temperature=1.0, min_p=0.2),
                                dict(temperature=0.9, top_k=40, top_p=0.8, min_p=0.05)])
@pytest.mark.parametrize("cluster,V", [(0, 3001), (1, 3001), (4, 3001), (8, 3002), (8, 3004), (None, 20012), (None, 20011)])
def test_sample_rows_draws_from_the_filtered_distribution(kw, cluster, V):
    """Both kernels (one block a row; a row over a cluster of 1 to 8 blocks), rows whose width is and is not a
    multiple of four, and the library's own choice for a wide row."""
    from synaptix_b200.ops import sampling as K
    R, seed = 64 if V < 8192 else 12, 1234
    x = torch.randn(R, V) * 2.5
    seq = torch.arange(R, dtype=torch.int32) % 7
    step = torch.arange(R, dtype=torch.int32)
    u_out = torch.empty(R, device="cuda")
    got = K.sample_rows(x.cuda(), kw.get("temperature", 1.0), kw.get("top_k", 0), kw.get("top_p", 1.0),
                        kw.get("min_p", 0.0), seed, seq.cuda(), step.cuda(), u_out=u_out, cluster=cluster).tolist()
    us = u_out.cpu().tolist()
    for r in range(R):
        u_ref = float(P.uniform_from_u32(P.philox_u32(seed, int(step[r]), int(seq[r]))))
        assert us[r] == u_ref
        v = P.processed_logits(x[r].numpy(), **kw)
        kept = np.isfinite(v)
        assert kept[got[r]], f"row {r}: token {got[r]} was filtered out"
        cum = P.multinomial_intervals(v)
        lo = cum[got[r] - 1] if got[r] > 0 else 0.0
        assert lo - 1e-4 <= u_ref <= cum[got[r]] + 1e-4, f"row {r}: u={u_ref} outside [{lo}, {cum[got[r]]}]"


@pytest.mark.parametrize("cluster,V", [(0, 777), (2, 777), (8, 776), (None, 9000)])
def test_sample_rows_kept_sets_match_exactly(cluster, V):
    """With a point mass the draw is forced; with top_k=1 it is the argmax, whatever u is."""
    from synaptix_b200.ops import sampling as K
    x = torch.randn(8, V)
    z = torch.zeros(8, dtype=torch.int32).cuda()
    got = K.sample_rows(x.cuda(), 1.0, 1, 1.0, 0.0, 5, z, z, cluster=cluster).tolist()
    assert got == x.argmax(dim=1).tolist()
    got = K.sample_rows(x.cuda(), 1.0, 0, 1e-6, 0.0, 5, z, z, cluster=cluster).tolist()
    assert got == x.argmax(dim=1).tolist()
    got = K.sample_rows(x.cuda(), 1.0, 0, 1.0, 1.0, 5, z, z, cluster=cluster).tolist()
    assert got == x.argmax(dim=1).tolist()
    # ties at the cut-off are all kept, -inf and NaN never: 3 equal maxima far apart, top_k = 1
    y = torch.randn(8, V)
    y[:, 3] = y[:, V // 2] = y[:, V - 1] = 30.0
    y[:, 5] = float("nan")
    y[:, 7] = float("-inf")
    seq = torch.arange(8, dtype=torch.int32).cuda()
    seen = set()
    for s in range(6):
        got = K.sample_rows(y.cuda(), 0.5, 1, 1.0, 0.0, 11, seq, torch.full((8,), s, dtype=torch.int32).cuda(), cluster=cluster).tolist()
        assert set(got) <= {3, V // 2, V - 1}
        seen |= set(got)
    assert seen == {3, V // 2, V - 1}
    got = K.sample_rows(x.cuda(), 0.0, 0, 1.0, 0.0, 5, z, z).tolist()       # temperature 0: greedy
    assert got == x.argmax(dim=1).tolist()


@pytest.mark.parametrize("V", [1000, 151936])
def test_sampling_does_not_depend_on_batch_composition(V):
    from synaptix_b200.ops import sampling as K
    x = torch.randn(6, V) * 2
    seq = torch.tensor([3, 1, 4, 1, 5, 9], dtype=torch.int32)
    step = torch.tensor([2, 7, 1, 8, 2, 8], dtype=torch.int32)
    whole = K.sample_rows(x.cuda(), 0.8, 50, 0.9, 0.0, 99, seq.cuda(), step.cuda()).tolist()
    for r in range(6):
        one = K.sample_rows(x[r:r + 1].cuda(), 0.8, 50, 0.9, 0.0, 99, seq[r:r + 1].cuda(), step[r:r + 1].cuda()).tolist()
        assert one[0] == whole[r]


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(389, 32), (100, 256), (2560, 2560), (48, 9728), (16, 64)])
def test_skinny_gemm(M, N, K):
    from synaptix_b200.ops.decode import skinny_gemm
    g = torch.Generator().manual_seed(M * 1000 + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    for ks in (8, 16):
        out = skinny_gemm(x.cuda(), w.cuda(), epilogue="f32", ks=ks)
        assert out.shape == (M, N)
        assert torch.allclose(out.cpu().double(), ref, atol=2e-5 * math.sqrt(K), rtol=1e-5), f"ks={ks}"
    out = skinny_gemm(x.cuda(), w.cuda())
    assert out.dtype == torch.bfloat16 and torch.allclose(out.float().cpu().double(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M", [1, 8, 13, 16])
@pytest.mark.parametrize("I,K", [(9, 64), (160, 96), (1000, 2560)])
def test_skinny_gemm_silu_mul_epilogue(M, I, K):
    from synaptix_b200.ops.decode import skinny_gemm
    x = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(2 * I, K) * 2 / math.sqrt(K)).to(torch.bfloat16)
    y = x.double() @ w.double().T
    gate, up = y[:, :I], y[:, I:]
    ref = gate / (1 + torch.exp(-gate)) * up
    for ks in (8, 16):
        out = skinny_gemm(x.cuda(), w.cuda(), epilogue="silu_mul", ks=ks)
        assert out.shape == (M, I)
        assert torch.allclose(out.float().cpu().double(), ref, atol=3e-2, rtol=2e-2), f"ks={ks}"


def test_skinny_gemm_refuses_what_it_does_not_take():
    from synaptix_b200.ops import KernelError
    from synaptix_b200.ops.decode import skinny_gemm, skinny_supported
    w = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(KernelError, match="size"):               # the norm prologue: one or two rows
        skinny_gemm(None, w, norm_h=torch.zeros(3, 64, device="cuda"), norm_gain=torch.ones(64, device="cuda"))
    assert not skinny_supported(17, 64, 64, torch.bfloat16, torch.bfloat16)
    with pytest.raises(KernelError, match="size"):               # more than 16 rows
        skinny_gemm(torch.zeros(17, 64, dtype=torch.bfloat16, device="cuda"), w)
    with pytest.raises(KernelError, match="size"):               # 4 warps splitting K is not built
        skinny_gemm(torch.zeros(4, 64, dtype=torch.bfloat16, device="cuda"), w, ks=4)


@pytest.mark.parametrize("M", [1, 2])
@pytest.mark.parametrize("epilogue,N", [(None, 200), ("silu_mul", 144), ("f32", 389)])
@pytest.mark.parametrize("K", [320, 2560, 4096])
def test_skinny_gemm_with_norm_prologue(M, epilogue, N, K):
    from synaptix_b200.ops.decode import skinny_gemm
    h = torch.randn(M, K) * 2
    d = torch.randn(M, K).to(torch.bfloat16)
    gain = 1 + 0.2 * torch.randn(K)
    w = (torch.randn(N, K) / math.sqrt(K)).to(torch.bfloat16)
    s = h + d.float()
    xn = P.rms_norm(s, gain, 1e-5).to(torch.bfloat16)
    y = xn.double() @ w.double().T
    if epilogue == "silu_mul":
        gate, up = y[:, :N // 2], y[:, N // 2:]
        y = gate / (1 + torch.exp(-gate)) * up
    h_out = torch.full((M, K), float("nan"), device="cuda")
    out = skinny_gemm(None, w.cuda(), epilogue=epilogue, norm_h=h.cuda(), norm_delta=d.cuda(), norm_h_out=h_out,
                      norm_gain=gain.cuda(), norm_eps=1e-5, ks=8)
    assert torch.allclose(h_out.cpu(), s, atol=1e-6)
    assert torch.allclose(out.float().cpu().double(), y, atol=3e-2, rtol=2e-2)
    out = skinny_gemm(None, w.cuda(), epilogue=epilogue, norm_h=h.cuda(), norm_delta=None, norm_h_out=None,
                      norm_gain=gain.cuda(), norm_eps=1e-5)
    y2 = P.rms_norm(h, gain, 1e-5).to(torch.bfloat16).double() @ w.double().T
    if epilogue == "silu_mul":
        y2 = y2[:, :N // 2] / (1 + torch.exp(-y2[:, :N // 2])) * y2[:, N // 2:]
    assert torch.allclose(out.float().cpu().double(), y2, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("M", [1, 2, 5, 8, 13, 16])
@pytest.mark.parametrize("N,K", [(2560, 4096), (176, 96), (100, 320), (24, 9728)])
def test_skinny_gemm_adds_into_the_residual_and_prepares_the_norm(M, N, K):
    """h += x W^T in place, x~ = bf16(h * gain) and partial sums of squares of h; then a second product takes x~
    and the partial sums and must give what it gives for the plain rmsnorm(h) * gain (all three epilogues)."""
    from synaptix_b200.ops.decode import skinny_gemm_residual, skinny_gemm_scaled
    g = torch.Generator().manual_seed(M * 7919 + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    h0 = torch.randn(M, N, generator=g) * torch.logspace(-1, 1, M)[:, None]      # rows of very different size
    gain = 1 + 0.3 * torch.randn(N, generator=g)
    eps = 1e-5
    h_ref = h0.double() + x.double() @ w.double().T
    for ks in (8, 16):
        h = h0.clone().cuda()
        xt, ssq = skinny_gemm_residual(x.cuda(), w.cuda(), h, gain.cuda(), ks=ks)
        assert torch.allclose(h.cpu().double(), h_ref, atol=2e-5 * math.sqrt(K), rtol=1e-5), f"ks={ks}"
        assert ssq.shape == (M, (N + 15) // 16)
        assert torch.allclose(ssq.sum(1).cpu().double(), (h_ref ** 2).sum(1), rtol=1e-4), f"ks={ks}"
        assert torch.allclose(xt.float().cpu().double(), h_ref * gain.double(), atol=1e-3, rtol=1e-2), f"ks={ks}"
    # the consumer: N is its inner size now
    if N % 32:
        return
    xn = P.rms_norm(h.cpu(), gain, eps)
    for epilogue, N2 in ((None, 200), ("f32", 389), ("silu_mul", 144)):
        w2 = (torch.randn(N2, N, generator=g) / math.sqrt(N)).to(torch.bfloat16)
        y = xn.double() @ w2.double().T
        if epilogue == "silu_mul":
            y = y[:, :N2 // 2] / (1 + torch.exp(-y[:, :N2 // 2])) * y[:, N2 // 2:]
        for ks in (8, 16):
            out = skinny_gemm_scaled(xt, w2.cuda(), ssq, eps, epilogue=epilogue, ks=ks)
            assert torch.allclose(out.float().cpu().double(), y, atol=3e-2, rtol=2e-2), f"{epilogue} ks={ks}"
    out = skinny_gemm_scaled(xt, w2.cuda(), None, 0.0, epilogue="f32")          # without partial sums: a plain product
    assert torch.allclose(out.cpu().double(), xt.float().cpu().double() @ w2.double().T, atol=2e-5 * math.sqrt(N) * 30, rtol=1e-4)


def fast_attention_case(nh, nkv, hd, window, past, new, seed, scale=None):
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(seed)
    ks = [torch.randn(p + n, nkv, hd, generator=g).to(dtype).float() for p, n in zip(past, new)]
    vs = [torch.randn(p + n, nkv, hd, generator=g).to(dtype).float() for p, n in zip(past, new)]
    kp, vp, bt = make_paged(ks, vs, nkv, hd, dtype, seed=seed)
    T = sum(new)
    q = torch.randn(T, nh, hd, generator=g).to(dtype)
    pos = torch.cat([torch.arange(p, p + n) for p, n in zip(past, new)]).to(torch.int32)
    sot = torch.cat([torch.full((n,), i) for i, n in enumerate(new)]).to(torch.int32)
    scale = 1 / math.sqrt(hd) if scale is None else scale
    ref = attention_reference(q.float(), ks, vs, pos, sot, scale, window)
    return q, kp, vp, bt, pos, sot, scale, ref


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 128, None), (32, 8, 128, None), (6, 2, 32, None), (5, 1, 64, 24),
                                               (8, 8, 64, None), (16, 1, 128, 100), (3, 3, 32, 65)])
def test_attention_decode_kernel(nh, nkv, hd, window):
    from synaptix_b200.ops.attention import attn_decode
    past, new = [0, 130, 1000, 63, 64, 255], [1] * 6
    q, kp, vp, bt, pos, sot, scale, ref = fast_attention_case(nh, nkv, hd, window, past, new, 3)
    lens = torch.tensor([p + 1 for p in past], dtype=torch.int32).cuda()
    for n_splits in (1, 2, 5, 16, 37):
        for fused in (True, False, True):          # fused twice: the counters must be left at zero
            out = attn_decode(q.view(6, nh * hd).cuda(), kp, vp, lens, bt, nh, nkv, hd, scale, window, n_splits,
                              fused_merge=fused)
            err = (out.float().cpu().view(6, nh, hd) - ref).abs().max().item()
            assert err < 2e-2, f"n_splits={n_splits} fused={fused}: {err}"


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 128, None), (32, 8, 128, None), (6, 2, 32, None), (5, 1, 64, 24),
                                               (8, 8, 64, None), (16, 1, 128, 100), (3, 3, 32, 65)])
def test_attention_decode_kernel_with_pages_by_tma(nh, nkv, hd, window):
    """Split counts from one (a block sees all pages, its warps take them in turn) to more splits than pages; the
    cache's unused places hold NaN and the output starts as NaN, so that a value read from a place nobody wrote, or
    a row nobody wrote, shows."""
    from synaptix_b200.ops.attention import attn_decode_status, attn_decode_tma
    if hd == 32:
        pytest.skip("head size 32 stays on the cp.async kernel")
    past, new = [0, 130, 1000, 63, 64, 255, 4, 700], [1] * 8
    q, kp, vp, bt, pos, sot, scale, ref = fast_attention_case(nh, nkv, hd, window, past, new, 3)
    lens = torch.tensor([p + 1 for p in past], dtype=torch.int32).cuda()
    # 2, 4, 8, 16 splits merge among themselves as a cluster; the others, and those with cluster=False, through scratch
    for n_splits, cluster in [(1, None), (2, True), (3, None), (4, True), (5, None), (8, True), (16, True), (37, None),
                              (4, False), (16, False)]:
        out = torch.full((8, nh * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        attn_decode_tma(q.view(8, nh * hd).cuda(), kp, vp, lens, bt, nh, nkv, hd, scale, window, n_splits, out=out,
                        cluster=cluster)
        err = (out.float().cpu().view(8, nh, hd) - ref).abs().max().item()
        assert err < 2e-2, f"splits={n_splits} cluster={cluster}: {err}"
    torch.cuda.synchronize()
    assert attn_decode_status() == 0


@pytest.mark.parametrize("nh,nkv,hd,window,rot,norm", [(4, 2, 128, None, True, True), (32, 8, 128, None, True, True),
                                                        (6, 2, 32, None, True, False), (5, 1, 64, 24, False, True),
                                                        (8, 8, 64, None, True, True), (16, 1, 128, 100, False, False),
                                                        (3, 3, 32, 65, True, True)])
def test_attention_decode_kernel_that_prepares_the_heads(nh, nkv, hd, window, rot, norm):
    """From the raw fused projection: the kernel's output equals attention over (cache + the prepared new key and
    value), the cache holds the new key and value afterwards and nothing else moved; a second pass that only reads
    the cache (write_cache=False) gives the same output.  New tokens at a page's first, last and middle place."""
    from synaptix_b200.ops.attention import attn_decode_prep
    from synaptix_b200.parts import rotary_inv_freq
    dtype = torch.bfloat16
    past = [0, 130, 1000, 63, 64, 255]
    S = len(past)
    eps, theta = 1e-5, 30000.0
    g = torch.Generator().manual_seed(11)
    qkv = torch.randn(S, (nh + 2 * nkv) * hd, generator=g).to(dtype)
    wq, wk = 1 + 0.3 * torch.randn(hd, generator=g), 1 + 0.3 * torch.randn(hd, generator=g)
    pos = torch.tensor(past)
    x = qkv.float()
    q = x[:, :nh * hd].view(S, nh, hd)
    k_new = x[:, nh * hd:(nh + nkv) * hd].view(S, nkv, hd)
    v_new = x[:, (nh + nkv) * hd:].view(S, nkv, hd)
    if norm:
        q, k_new = P.rms_norm(q, wq, eps), P.rms_norm(k_new, wk, eps)
    if rot:
        f = P.rotary_freqs(theta, hd)
        q, k_new = P.rope_rotate_half(q, pos, f), P.rope_rotate_half(k_new, pos, f)
    q, k_new, v_new = q.to(dtype).float(), k_new.to(dtype).float(), v_new.to(dtype).float()
    ks = [torch.cat([torch.randn(p, nkv, hd, generator=g).to(dtype).float(), k_new[i:i + 1]]) for i, p in enumerate(past)]
    vs = [torch.cat([torch.randn(p, nkv, hd, generator=g).to(dtype).float(), v_new[i:i + 1]]) for i, p in enumerate(past)]
    scale = 1 / math.sqrt(hd)
    ref = attention_reference(q, ks, vs, pos.to(torch.int32), torch.arange(S, dtype=torch.int32), scale, window)
    # the cache WITHOUT the new tokens (their places hold NaN, like everything unwritten)
    kp, vp, bt = make_paged(ks, vs, nkv, hd, dtype, seed=5)
    for i, p in enumerate(past):
        page = int(bt[i, p // 64])
        kp[page, :, p % 64] = float("nan")
        vp[page, :, p % 64] = float("nan")
    before_k, before_v = kp.clone(), vp.clone()
    lens = torch.tensor([p + 1 for p in past], dtype=torch.int32).cuda()
    inv = torch.from_numpy(rotary_inv_freq(theta, hd)).cuda() if rot else None
    gq, gk = (wq.cuda(), wk.cuda()) if norm else (None, None)
    for n_splits in (1, 3, 16):
        kp.copy_(before_k); vp.copy_(before_v)
        out = attn_decode_prep(qkv.cuda(), kp, vp, lens, bt, nh, nkv, hd, scale, window, n_splits, gq, gk, inv, eps, True)
        err = (out.float().cpu().view(S, nh, hd) - ref).abs().max().item()
        assert err < 2e-2, f"n_splits={n_splits}: {err}"
        kc, vc, bc = kp.float().cpu(), vp.float().cpu(), bt.cpu()
        changed = torch.zeros(kc.shape[0], 64, dtype=torch.bool)
        for i, p in enumerate(past):
            page = int(bc[i, p // 64])
            assert torch.allclose(kc[page, :, p % 64], k_new[i], atol=2e-2, rtol=2e-2)
            assert torch.equal(vc[page, :, p % 64], v_new[i])
            changed[page, p % 64] = True
        same = lambda a, b: torch.equal(torch.nan_to_num(a.float().cpu(), nan=12345.0), torch.nan_to_num(b.float().cpu(), nan=12345.0))
        keep = ~changed[:, None, :, None].expand_as(kc)
        assert same(torch.where(keep, kp.float().cpu(), torch.zeros(())), torch.where(keep, before_k.float().cpu(), torch.zeros(())))
        assert same(torch.where(keep, vp.float().cpu(), torch.zeros(())), torch.where(keep, before_v.float().cpu(), torch.zeros(())))
        # the cache now holds the tokens: a pass that writes nothing must see them there
        again = attn_decode_prep(qkv.cuda(), kp, vp, lens, bt, nh, nkv, hd, scale, window, n_splits, gq, gk, inv, eps, False)
        assert (again.float() - out.float()).abs().max().item() < 1e-2
    # the same through the kernel that brings pages by TMA (head size 64 and 128)
    if hd == 32:
        return
    from synaptix_b200.ops.attention import attn_decode_tma
    for n_splits in (1, 3, 4, 16):                         # 4: the splits merge as a cluster
        kp.copy_(before_k); vp.copy_(before_v)
        out = attn_decode_tma(qkv.cuda(), kp, vp, lens, bt, nh, nkv, hd, scale, window, n_splits, prep=True, wq=gq, wk=gk,
                              inv_freq=inv, eps=eps, write_cache=True)
        err = (out.float().cpu().view(S, nh, hd) - ref).abs().max().item()
        assert err < 2e-2, f"tma splits={n_splits}: {err}"
        kc, vc, bc = kp.float().cpu(), vp.float().cpu(), bt.cpu()
        changed = torch.zeros(kc.shape[0], 64, dtype=torch.bool)
        for i, p in enumerate(past):
            page = int(bc[i, p // 64])
            assert torch.allclose(kc[page, :, p % 64], k_new[i], atol=2e-2, rtol=2e-2)
            assert torch.equal(vc[page, :, p % 64], v_new[i])
            changed[page, p % 64] = True
        keep = ~changed[:, None, :, None].expand_as(kc)
        assert same(torch.where(keep, kp.float().cpu(), torch.zeros(())), torch.where(keep, before_k.float().cpu(), torch.zeros(())))
        assert same(torch.where(keep, vp.float().cpu(), torch.zeros(())), torch.where(keep, before_v.float().cpu(), torch.zeros(())))
        again = attn_decode_tma(qkv.cuda(), kp, vp, lens, bt, nh, nkv, hd, scale, window, n_splits, prep=True, wq=gq, wk=gk,
                                inv_freq=inv, eps=eps, write_cache=False)
        assert (again.float() - out.float()).abs().max().item() < 1e-2




def test_fast_attention_finds_one_far_key_and_respects_the_window_edge():
    from synaptix_b200.ops.attention import attn_decode, attn_decode_tma, attn_prefill, query_tiles
    nh, nkv, hd = 4, 2, 64
    dt = torch.bfloat16
    dev = lambda x: torch.tensor(x, dtype=torch.int32).cuda()
    for L, far, W in [(700, 0, None), (700, 333, None), (700, 699, None), (700, 63, None), (700, 64, None),
                      (200, 130, 70), (134, 64, 70), (71, 1, 70)]:
        k = torch.randn(L, nkv, hd) * 0.1
        v = torch.randn(L, nkv, hd)
        q = torch.randn(1, nh, hd)
        q[0, 1], q[0, 3] = q[0, 0].clone(), q[0, 2].clone()
        for kh in range(nkv):
            k[far, kh] = q[0, kh * 2] / q[0, kh * 2].norm() * 40.0
            if W is not None and far - 1 >= 0:          # far is the window's first key; the one before it must not count
                assert far == L - W
                k[far - 1, kh] = q[0, kh * 2] / q[0, kh * 2].norm() * 80.0
                v[far - 1, kh] = 1000.0
        kp, vp, bt = make_paged([k], [v], nkv, hd, dt, seed=L + far)
        qd = q.view(1, nh * hd).to(dt).cuda()
        want = torch.stack([v[far, h // 2].to(dt).float() for h in range(nh)])
        for n_splits in (1, 3):
            out = attn_decode(qd, kp, vp, dev([L]), bt, nh, nkv, hd, 1.0, W, n_splits).float().cpu().view(nh, hd)
            assert torch.allclose(out, want, atol=2e-2), f"decode L={L} far={far} W={W} splits={n_splits}"
        for n_splits in (1, 3):
            out = attn_decode_tma(qd, kp, vp, dev([L]), bt, nh, nkv, hd, 1.0, W, n_splits).float().cpu().view(nh, hd)
            assert torch.allclose(out, want, atol=2e-2), f"decode, pages by TMA, L={L} far={far} W={W} splits={n_splits}"
        out = attn_prefill(qd, kp, vp, dev([0]), dev([0]), dev([0, 1]), dev([L - 1]), dev([L]), bt, nh, nkv, hd, 1.0, W)
        assert torch.allclose(out.float().cpu().view(nh, hd), want, atol=2e-2), f"prefill L={L} far={far} W={W}"


def test_tcgen05_attention_finds_one_far_key_and_respects_the_window_edge():
    """One key among hundreds carries the whole weight; with a window, the key just before its edge would win if
    it counted.  The last query of a sequence held in the cache, as a one-row prompt step."""
    from synaptix_b200.ops.attention import attn_prefill_tc
    nh, nkv, hd = 4, 2, 128
    dt = torch.bfloat16
    dev = lambda x: torch.tensor(x, dtype=torch.int32).cuda()
    for L, far, W in [(700, 0, None), (700, 333, None), (700, 699, None), (700, 127, None), (700, 128, None),
                      (200, 130, 70), (134, 64, 70), (71, 1, 70), (300, 128, 172)]:
        k = torch.randn(L, nkv, hd) * 0.1
        v = torch.randn(L, nkv, hd)
        q = torch.randn(1, nh, hd)
        q[0, 1], q[0, 3] = q[0, 0].clone(), q[0, 2].clone()
        for kh in range(nkv):
            k[far, kh] = q[0, kh * 2] / q[0, kh * 2].norm() * 40.0
            if W is not None and far - 1 >= 0:
                assert far == L - W
                k[far - 1, kh] = q[0, kh * 2] / q[0, kh * 2].norm() * 80.0
                v[far - 1, kh] = 1000.0
        kp, vp, bt = make_paged([k], [v], nkv, hd, dt, seed=L + far)
        qd = q.view(1, nh * hd).to(dt).cuda()
        want = torch.stack([v[far, h // 2].to(dt).float() for h in range(nh)])
        out = attn_prefill_tc(qd, kp, vp, dev([0]), dev([0]), dev([0, 1]), dev([L - 1]), dev([L]), bt, nh, nkv, hd, 1.0, W)
        assert torch.allclose(out.float().cpu().view(nh, hd), want, atol=2e-2), f"L={L} far={far} W={W}"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (65, 256, 2560), (200, 300, 72), (1000, 389, 96), (130, 24, 8),
                                    (2048, 1024, 2560), (513, 2560, 1224)])
def test_gemm_tc(M, N, K):
    """The tcgen05 product against float64, at sizes with ragged edges in M, N and K."""
    from synaptix_b200.ops.gemm_tc import gemm_tc, gemm_tc_status
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    out = gemm_tc(x.cuda(), w.cuda(), epilogue="f32")
    assert torch.allclose(out.cpu().double(), ref, atol=2e-5 * math.sqrt(K), rtol=1e-5)
    out = gemm_tc(x.cuda(), w.cuda())
    assert out.dtype == torch.bfloat16 and torch.allclose(out.float().cpu().double(), ref, atol=2e-2, rtol=2e-2)
    assert gemm_tc_status() == 0


@pytest.mark.parametrize("M,N,K,epilogue,is_cut", [
    # a nearly empty last round of whole tiles: its tiles are cut, the blocks add up inside the kernel
    (2048, 2560, 4096, "f32", True), (2048, 2560, 9728, None, True), (2000, 2500, 4104, "f32", True), (1300, 3484, 3656, None, True),
    (2048, 2560, 512, None, False), (1024, 6144, 2560, None, False),
    # one row of tiles, at least half as many as SMs: all tiles cut, a second kernel adds up
    (64, 19456, 2560, "silu_mul", True), (100, 20000, 136, None, True), (33, 30000, 264, "f32", True), (17, 25000, 200, "silu_mul", True),
    # several rows of tiles, fewer than the SMs, long K: all tiles cut into shares that may begin and end inside a tile
    (512, 2560, 4096, None, True), (300, 2560, 9728, "f32", True), (640, 2500, 4104, "f32", True), (400, 1024, 3080, None, True),
    (384, 2048, 6144, "silu_mul", True), (512, 6144, 2560, None, False),
    # a handful of tiles: the two-kernel split form
    (64, 6144, 2560, None, False), (64, 2560, 4096, "f32", False), (17, 389, 96, "f32", False), (128, 256, 64, "f32", False),
    (200, 700, 1224, "silu_mul", False), (40, 24, 8, "f32", False)])
def test_gemm_tc_tiles_cut_over_k(M, N, K, epilogue, is_cut):
    """Shapes whose tiles do not fill a round of all SMs: the persistent kernel cuts them over K and the blocks
    of a tile add their partial tiles up.  The result must be the product everywhere, for ragged M, N and K,
    and the same bits twice (the order of addition is fixed)."""
    from synaptix_b200.ops.gemm_tc import gemm_tc, gemm_tc_status, plan_stream
    n_whole, n_cut, zmax, grid = plan_stream(M, N, K, epilogue)
    assert (n_cut > 0) == is_cut, "what this GPU's SM count makes of the shape"
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * (2 if epilogue == "silu_mul" else 1) / math.sqrt(K)).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    if epilogue == "silu_mul":
        ref = ref[:, :N // 2] / (1 + torch.exp(-ref[:, :N // 2])) * ref[:, N // 2:]
    tol = dict(atol=2e-5 * math.sqrt(K), rtol=1e-5) if epilogue == "f32" else dict(atol=3e-2, rtol=2e-2)
    out = torch.full(ref.shape, float("nan"), dtype=torch.float32 if epilogue == "f32" else torch.bfloat16, device="cuda")
    gemm_tc(x.cuda(), w.cuda(), epilogue=epilogue, out=out)
    assert torch.allclose(out.float().cpu().double(), ref, **tol)
    again = gemm_tc(x.cuda(), w.cuda(), epilogue=epilogue)
    assert torch.equal(again, out)
    whole = gemm_tc(x.cuda(), w.cuda(), epilogue=epilogue, cut=False, splits=1)
    assert torch.allclose(whole.float().cpu().double(), ref, **tol)
    assert gemm_tc_status() == 0


@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (77, 160, 200), (300, 1000, 2560), (2048, 129, 96)])
def test_gemm_tc_silu_mul_epilogue(M, I, K):
    from synaptix_b200.ops.gemm_tc import gemm_tc, gemm_tc_status
    x = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(2 * I, K) * 2 / math.sqrt(K)).to(torch.bfloat16)
    y = x.double() @ w.double().T
    ref = y[:, :I] / (1 + torch.exp(-y[:, :I])) * y[:, I:]
    out = gemm_tc(x.cuda(), w.cuda(), epilogue="silu_mul")
    assert out.shape == (M, I) and torch.allclose(out.float().cpu().double(), ref, atol=3e-2, rtol=2e-2)
    assert gemm_tc_status() == 0


@pytest.mark.parametrize("M,N,K,epilogue", [(64, 2560, 4096, None), (17, 389, 96, "f32"), (64, 6144, 2560, None),
                                             (33, 320, 1224, "silu_mul"), (128, 256, 64, "f32"), (40, 2560, 9728, "f32")])
def test_gemm_tc_split_k(M, N, K, epilogue):
    """Few rows: K split over blocks, float32 partial tiles added in a fixed order by a second kernel."""
    from synaptix_b200.ops.gemm_tc import gemm_tc, gemm_tc_status
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    if epilogue == "silu_mul":
        ref = ref[:, :N // 2] / (1 + torch.exp(-ref[:, :N // 2])) * ref[:, N // 2:]
    outs = []
    for splits in (None, 2, 3, 7, 1000):
        out = gemm_tc(x.cuda(), w.cuda(), epilogue=epilogue, splits=splits)
        tol = dict(atol=2e-5 * math.sqrt(K), rtol=1e-5) if epilogue == "f32" else dict(atol=3e-2, rtol=2e-2)
        assert torch.allclose(out.float().cpu().double(), ref, **tol), f"splits={splits}"
        outs.append(out)
    again = gemm_tc(x.cuda(), w.cuda(), epilogue=epilogue, splits=3)
    assert torch.equal(again, outs[2])                  # the order of addition is fixed
    assert gemm_tc_status() == 0


@pytest.mark.parametrize("M", [1, 17, 40, 64, 100, 128, 129, 150, 200, 256])
@pytest.mark.parametrize("N,K", [(2560, 4096), (389, 96), (264, 72), (130, 64), (1000, 1224)])
def test_gemm_ws(M, N, K):
    """The weight-streaming tcgen05 product (weights as the M side, K shared by a cluster's blocks) against
    float64: ragged M, N and K, every number of blocks a cluster may have, all plain epilogues, with and without
    row factors; and the same bits twice (the blocks add up in a fixed order)."""
    from synaptix_b200.ops.gemm_ws import gemm_ws, gemm_ws_status, plan_ws
    g = torch.Generator().manual_seed(M * 31 + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 2 / math.sqrt(K)).to(torch.bfloat16)
    ssq = torch.rand(M, 5, generator=g) * K * torch.logspace(-1, 1, M)[:, None]
    eps = 1e-5
    rf = torch.rsqrt(ssq.double().sum(1) / K + eps)[:, None]
    ref = x.double() @ w.double().T
    tiles, auto = plan_ws(M, N, K)
    assert tiles == (N + 127) // 128 and auto in (1, 2, 4, 8)
    xd, wd, sd = x.cuda(), w.cuda(), ssq.cuda()
    for splits in (None, 1, 2, 4, 8):
        out = gemm_ws(xd, wd, epilogue="f32", splits=splits)
        assert torch.allclose(out.cpu().double(), ref, atol=2e-5 * math.sqrt(K), rtol=1e-5), f"splits={splits}"
        assert torch.equal(out, gemm_ws(xd, wd, epilogue="f32", splits=splits))
        out = gemm_ws(xd, wd, splits=splits)
        assert out.dtype == torch.bfloat16 and torch.allclose(out.float().cpu().double(), ref, atol=3e-2, rtol=2e-2)
        out = gemm_ws(xd, wd, epilogue="f32", ssq=sd, eps=eps, splits=splits)
        assert torch.allclose(out.cpu().double(), ref * rf, atol=2e-5 * math.sqrt(K) * rf.max().item(), rtol=1e-4), f"splits={splits}"
        if N % 2 == 0:
            for s_, f_ in ((None, 1.0), (sd, rf)):
                y = ref * f_
                want = y[:, :N // 2] / (1 + torch.exp(-y[:, :N // 2])) * y[:, N // 2:]
                out = gemm_ws(xd, wd, epilogue="silu_mul", ssq=s_, eps=eps, splits=splits)
                assert out.shape == (M, N // 2)
                assert torch.allclose(out.float().cpu().double(), want, atol=3e-2, rtol=2e-2), f"silu splits={splits}"
    assert gemm_ws_status() == 0


@pytest.mark.parametrize("M", [3, 17, 64, 128, 144, 256])
@pytest.mark.parametrize("N,K", [(2560, 4096), (176, 96), (100, 320), (24, 9728)])
def test_gemm_ws_adds_into_the_residual_and_prepares_the_norm(M, N, K):
    """h += x W^T in place, x~ = bf16(h * gain) and partial sums of squares of h; then a second product takes x~
    and the partial sums and must give what it gives for the plain rmsnorm(h) * gain."""
    from synaptix_b200.ops.gemm_ws import gemm_ws, gemm_ws_residual, gemm_ws_status
    g = torch.Generator().manual_seed(M * 7919 + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    h0 = torch.randn(M, N, generator=g) * torch.logspace(-1, 1, M)[:, None]      # rows of very different size
    gain = 1 + 0.3 * torch.randn(N, generator=g)
    eps = 1e-5
    h_ref = h0.double() + x.double() @ w.double().T
    for splits in (None, 1, 2, 8):
        h = h0.clone().cuda()
        xt, ssq = gemm_ws_residual(x.cuda(), w.cuda(), h, gain.cuda(), splits=splits)
        assert torch.allclose(h.cpu().double(), h_ref, atol=2e-5 * math.sqrt(K), rtol=1e-5), f"splits={splits}"
        assert ssq.shape[0] == M and torch.isfinite(ssq).all()
        assert torch.allclose(ssq.sum(1).cpu().double(), (h_ref ** 2).sum(1), rtol=1e-4), f"splits={splits}"
        assert torch.allclose(xt.float().cpu().double(), h_ref * gain.double(), atol=1e-3, rtol=1e-2), f"splits={splits}"
    if N % 8:
        return
    xn = P.rms_norm(h.cpu(), gain, eps)
    for epilogue, N2 in ((None, 200), ("f32", 389), ("silu_mul", 144)):
        w2 = (torch.randn(N2, N, generator=g) / math.sqrt(N)).to(torch.bfloat16)
        y = xn.double() @ w2.double().T
        if epilogue == "silu_mul":
            y = y[:, :N2 // 2] / (1 + torch.exp(-y[:, :N2 // 2])) * y[:, N2 // 2:]
        out = gemm_ws(xt, w2.cuda(), epilogue=epilogue, ssq=ssq, eps=eps)
        assert torch.allclose(out.float().cpu().double(), y, atol=3e-2, rtol=2e-2), f"{epilogue}"
    assert gemm_ws_status() == 0


def test_gemm_ws_refuses_what_it_does_not_take():
    from synaptix_b200.ops import KernelError
    from synaptix_b200.ops.gemm_ws import gemm_ws
    x = torch.zeros(257, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(32, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(KernelError):
        gemm_ws(x, w)                                           # more than 256 rows
    with pytest.raises(KernelError):
        gemm_ws(x[:8, :60].contiguous(), w[:, :60].contiguous())   # K no multiple of 8
    with pytest.raises(KernelError):
        gemm_ws(x[:8], w, splits=3)
    with pytest.raises(KernelError):
        gemm_ws(x[:8].float(), w)
